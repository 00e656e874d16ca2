// Tensor-parallel decode epilogue in ONE kernel: all-reduce of the row-parallel partial outputs over NVLink peer
// memory, residual add, and the RMSNorm that feeds the next projection.
//
//   x[row] += sum_r partial_r[row]          (same summation order on every rank: bitwise identical x everywhere)
//   h[row]  = x[row] * rsqrt(mean(x^2) + eps) * w        (optional)
//
// Protocol: self-validating data, no flags and no barriers (the scheme usually called a Lamport all-reduce).
// Every rank owns three receive buffers [W sources][cap] in symmetric memory, pre-filled with a sentinel bit pattern
// (0x8000 per 16-bit lane: negative zero, which the sender rewrites to +0).  Call k pushes this rank's partial rows
// into slot (k mod 3, source = rank) of every peer with 16-byte stores, then polls its own slot k mod 3 until no
// lane of a vector is the sentinel; arrival of the data is the signal, so the latency is one NVLink store, not a
// flag round trip.  Call k also re-fills slot (k+2) mod 3: a peer can only be writing that slot in call k+2, which it
// cannot have entered before this rank pushed call k+1.  The call counter and the per-slot fill sizes live in device
// memory and are advanced by the last CTA to finish, so the launch is replayable from a CUDA graph.
// Polls are bounded by a globaltimer deadline; on expiry the status word is set and the CTA leaves.
//
// One CTA per row; a thread owns up to AR_VPT 16-byte vectors of the row in registers (row length <= 8*AR_VPT*1024).
//
// The reference has no tensor-parallel decode; its all-reduce is a host loop (src/gpu/multi_gpu.rs:583-700) and its
// RMSNorm a CPU loop (src/nn/normalization.rs:652, rms_normalize).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

constexpr int AR_VPT = 2;  // vectors per thread held in registers

__device__ __forceinline__ void ar_st_sys(void* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ar_ld_volatile(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ar_fix_word(unsigned w) {  // -0 -> +0 in both 16-bit lanes
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}
__device__ __forceinline__ bool ar_word_pending(unsigned w) { return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u; }
__device__ __forceinline__ bool ar_pending(const uint4& v) {
  return ar_word_pending(v.x) || ar_word_pending(v.y) || ar_word_pending(v.z) || ar_word_pending(v.w);
}

template <typename T> __device__ __forceinline__ float2 ar_unpack(unsigned w);
template <> __device__ __forceinline__ float2 ar_unpack<__half>(unsigned w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <> __device__ __forceinline__ float2 ar_unpack<__nv_bfloat16>(unsigned w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
template <typename T> __device__ __forceinline__ unsigned ar_pack(float a, float b);
template <> __device__ __forceinline__ unsigned ar_pack<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&h);
}
template <> __device__ __forceinline__ unsigned ar_pack<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&h);
}

template <typename T>
__device__ __forceinline__ void ar_accumulate(float (&acc)[8], const uint4& v) {
  const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = ar_unpack<T>(w[j]);
    acc[2 * j] += f.x;
    acc[2 * j + 1] += f.y;
  }
}

// state: int32[8] = {call counter, CTAs finished, fill[0], fill[1], fill[2], -, -, -}; fill[s] = vectors per source
// that the last call using slot s wrote.
template <typename T>
__global__ void __launch_bounds__(1024, 1) ar_residual_norm_kernel(const ArNormArgs a) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int W = a.world, R = a.rank;
  const int row = blockIdx.x;
  const int vpr = a.d / 8;                         // vectors per row
  volatile int* state = a.state;
  const int call = state[0];
  const int slot = call % 3, clear_slot = (call + 2) % 3;
  const long long cap_v = a.cap_numel / 8;         // vectors per source region
  uint4* mine = reinterpret_cast<uint4*>(a.bufs[R]);
  const uint4 sentinel = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);

  // ---- push this rank's partial row to every peer (and keep it in registers)
  uint4 own[AR_VPT];
#pragma unroll
  for (int t = 0; t < AR_VPT; ++t) {
    const int i = threadIdx.x + t * blockDim.x;
    if (i < vpr) {
      uint4 v = reinterpret_cast<const uint4*>(a.partial)[(long long)row * vpr + i];
      v.x = ar_fix_word(v.x); v.y = ar_fix_word(v.y); v.z = ar_fix_word(v.z); v.w = ar_fix_word(v.w);
      own[t] = v;
      const long long off = ((long long)slot * W + R) * cap_v + (long long)row * vpr + i;
      for (int s = 1; s < W; ++s) {
        const int p = (R + s) % W;
        ar_st_sys(reinterpret_cast<uint4*>(a.bufs[p]) + off, v);
      }
    }
  }
  // ---- re-arm the slot that call + 2 will use
  if (W > 1) {
    const long long fill = state[2 + clear_slot];
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < fill; v += (long long)gridDim.x * blockDim.x)
      for (int r = 0; r < W; ++r)
        if (r != R) mine[((long long)clear_slot * W + r) * cap_v + v] = sentinel;
  }
  // ---- wait for the peers' rows, sum in rank order, add the residual
  bool ok = true;
  const unsigned long long t0 = globaltimer_ns();
  float ss = 0.f;
  uint4 xnew[AR_VPT];
#pragma unroll
  for (int t = 0; t < AR_VPT; ++t) {
    const int i = threadIdx.x + t * blockDim.x;
    if (i < vpr) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int r = 0; r < W; ++r) {
        uint4 v = own[t];
        if (r != R) {
          const uint4* src = mine + ((long long)slot * W + r) * cap_v + (long long)row * vpr + i;
          unsigned it = 0;
          v = ar_ld_volatile(src);
          while (ok && ar_pending(v)) {
            if ((++it & 0xff) == 0 && globaltimer_ns() - t0 > a.timeout_ns) {
              atomicCAS(a.status, 0, RT_ERR_TIMEOUT_PEER);
              ok = false;
            }
            v = ar_ld_volatile(src);
          }
        }
        ar_accumulate<T>(acc, v);
      }
      uint4 xv = reinterpret_cast<const uint4*>(a.x)[(long long)row * vpr + i];
      const unsigned xw[4] = {xv.x, xv.y, xv.z, xv.w};
      unsigned ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = ar_unpack<T>(xw[j]);
        const unsigned pk = ar_pack<T>(f.x + acc[2 * j], f.y + acc[2 * j + 1]);
        ow[j] = pk;
        const float2 g = ar_unpack<T>(pk);    // the norm sees the rounded residual stream, as a separate kernel would
        ss += g.x * g.x + g.y * g.y;
      }
      xnew[t] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      reinterpret_cast<uint4*>(a.x)[(long long)row * vpr + i] = xnew[t];
    }
  }
  // ---- RMSNorm of the new residual stream
  if (a.h != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (threadIdx.x == 0) red[0] = rsqrtf(v / (float)a.d + a.eps);
    }
    __syncthreads();
    const float rstd = red[0];
#pragma unroll
    for (int t = 0; t < AR_VPT; ++t) {
      const int i = threadIdx.x + t * blockDim.x;
      if (i < vpr) {
        const uint4 wv = reinterpret_cast<const uint4*>(a.w)[i];
        const unsigned xw[4] = {xnew[t].x, xnew[t].y, xnew[t].z, xnew[t].w};
        const unsigned ww[4] = {wv.x, wv.y, wv.z, wv.w};
        unsigned ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = ar_unpack<T>(xw[j]), g = ar_unpack<T>(ww[j]);
          ow[j] = ar_pack<T>(f.x * rstd * g.x, f.y * rstd * g.y);
        }
        reinterpret_cast<uint4*>(a.h)[(long long)row * vpr + i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
  }
  // ---- the last CTA to finish advances the call counter (every CTA has read it by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.state + 1, 1);
    if (done == (int)gridDim.x - 1) {
      state[1] = 0;
      state[2 + slot] = (int)((long long)gridDim.x * vpr);
      __threadfence();
      state[0] = call + 1;
    }
  }
}

}  // namespace

void ar_residual_norm(const ArNormArgs& a, cudaStream_t stream) {
  RT_CHECK(a.world >= 1 && a.world <= RT_MAX_PEERS && a.rank >= 0 && a.rank < a.world, "ar_residual_norm: bad world / rank");
  RT_CHECK(a.dtype == DT_F16 || a.dtype == DT_BF16, "ar_residual_norm: fp16 or bf16 activations");
  RT_CHECK(a.d % 8 == 0 && a.d / 8 <= AR_VPT * 1024, "ar_residual_norm: row length must be a multiple of 8, at most 16384");
  RT_CHECK(a.rows >= 1 && (long long)a.rows * a.d <= a.cap_numel && a.cap_numel % 8 == 0,
           "ar_residual_norm: rows * d exceeds the receive buffers");
  RT_CHECK(a.state != nullptr && a.partial != nullptr && a.x != nullptr, "ar_residual_norm: null operand");
  RT_CHECK(a.h == nullptr || a.w != nullptr, "ar_residual_norm: norm weight required with a norm output");
  const int vpr = a.d / 8;
  const int threads = std::min(1024, std::max(32, ((vpr + 31) / 32) * 32));
  ArNormArgs b = a;
  b.status = status_word(current_device());
  if (a.dtype == DT_F16) launch_pdl(ar_residual_norm_kernel<__half>, dim3(a.rows), dim3(threads), 0, stream, b);
  else launch_pdl(ar_residual_norm_kernel<__nv_bfloat16>, dim3(a.rows), dim3(threads), 0, stream, b);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
