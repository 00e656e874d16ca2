// Dequant-fused matrix-vector products for GGUF Q4_0 / Q8_0 weights (decode path, small batch):
//
//   y[m][n] = sum_k dequant(W)[n][k] * x[m][k]  (+ bias[n]) (+ residual[m][n])      m < M <= 8 per launch
//
// The weights stay quantised in HBM (0.5625 B / weight for Q4_0) and are expanded in registers, so a
// decode step streams each weight byte exactly once.  One warp owns one output row n; lane l walks the
// 32-weight blocks l, l+32, ... of that row (coalesced 16-byte loads of the nibbles, 2-byte loads of the
// scales), multiplies them against fp16 activations read through L1, accumulates each block in half2
// and the running sum in fp32, and a warp shuffle finishes the row.
//
// Device layout ("repacked" once at load from the GGUF block stream, same information, same size):
//   Q4_0: qs [N][K/32] uint4  - word i of a block holds weights 8i..8i+7 with weight 8i+2j in bits
//                               [4j, 4j+4) and weight 8i+2j+1 in bits [16+4j, 20+4j), so that
//                               ((w >> 4j) & 0x000F000F) | 0x64006400 is the half2 (1024+q_even, 1024+q_odd)
//         d  [N][K/32] half   - block scales
//   Q8_0: qs [N][K/32][32] int8 (natural order), d as above.
// GGUF stores Q4_0 as f16 d + 16 bytes with weight j in the low and weight j+16 in the high nibble of
// byte j (block layout per the GGUF spec; the reference only records the block sizes,
// example-cli/src/model/formats/gguf.rs:131-135, and never decodes them, tensor_loader.rs:103-122).
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

// Expand one repacked Q4_0 block (4 words) into 16 half2 of (q - 8).
__device__ __forceinline__ void expand_q4(const uint4& q, __half2 (&w)[16]) {
  const uint32_t words[4] = {q.x, q.y, q.z, q.w};
  const __half2 bias = __half2half2(__ushort_as_half(0x6408));  // 1032
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t bits = ((words[i] >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
      w[i * 4 + j] = __hsub2(*reinterpret_cast<const __half2*>(&bits), bias);
    }
  }
}

__device__ __forceinline__ void expand_q8(const int8_t* q, __half2 (&w)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(q);
  const uint4 b = *reinterpret_cast<const uint4*>(q + 16);
  const uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v0 = (int)(int8_t)(words[i] & 0xFF), v1 = (int)(int8_t)((words[i] >> 8) & 0xFF);
    const int v2 = (int)(int8_t)((words[i] >> 16) & 0xFF), v3 = (int)(int8_t)(words[i] >> 24);
    w[2 * i] = __halves2half2(__int2half_rn(v0), __int2half_rn(v1));
    w[2 * i + 1] = __halves2half2(__int2half_rn(v2), __int2half_rn(v3));
  }
}

// Q8 = false: Q4_0, true: Q8_0.  M rows of x handled together (dequant shared between them).
template <bool Q8, int M>
__global__ void __launch_bounds__(256) q_gemv_kernel(const void* __restrict__ qs,
                                                     const __half* __restrict__ scales,
                                                     const __half* __restrict__ x, long long ldx,
                                                     __half* __restrict__ y, long long ldy,
                                                     const __half* __restrict__ bias,
                                                     const __half* __restrict__ residual, long long ldr,
                                                     int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int nb = K >> 5;  // blocks per row
  const __half* drow = scales + (long long)n * nb;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;

  for (int b = lane; b < nb; b += 32) {
    __half2 w[16];
    if (Q8) {
      expand_q8(reinterpret_cast<const int8_t*>(qs) + ((long long)n * nb + b) * 32, w);
    } else {
      expand_q4(reinterpret_cast<const uint4*>(qs)[(long long)n * nb + b], w);
    }
    const float d = __half2float(drow[b]);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4* xp = reinterpret_cast<const uint4*>(x + m * ldx + (b << 5));
      __half2 s = __float2half2_rn(0.f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 xv = __ldg(xp + i);
        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) s = __hfma2(w[i * 4 + j], xh[j], s);
      }
      const float2 f = __half22float2(s);
      acc[m] = fmaf(d, f.x + f.y, acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float v = warp_sum_f(acc[m]);
    if (lane == 0) {
      if (bias) v += __half2float(bias[n]);
      if (residual) v += __half2float(residual[m * ldr + n]);
      y[m * ldy + n] = __float2half(v);
    }
  }
}

template <bool Q8>
static void launch_rows(const QGemvArgs& a, int m0, int m, cudaStream_t s) {
  const int warps = 8;
  const dim3 grid((a.N + warps - 1) / warps), block(warps * 32);
  const __half* x = reinterpret_cast<const __half*>(a.x) + (long long)m0 * a.ldx;
  __half* y = reinterpret_cast<__half*>(a.y) + (long long)m0 * a.ldy;
  const __half* r = a.residual ? reinterpret_cast<const __half*>(a.residual) + (long long)m0 * a.ldr : nullptr;
  auto sc = reinterpret_cast<const __half*>(a.scales);
  auto bi = reinterpret_cast<const __half*>(a.bias);
#define RT_QG(MM) q_gemv_kernel<Q8, MM><<<grid, block, 0, s>>>(a.qs, sc, x, a.ldx, y, a.ldy, bi, r, a.ldr, a.N, a.K)
  switch (m) {
    case 1: RT_QG(1); break;
    case 2: RT_QG(2); break;
    case 3: RT_QG(3); break;
    case 4: RT_QG(4); break;
    case 5: RT_QG(5); break;
    case 6: RT_QG(6); break;
    case 7: RT_QG(7); break;
    default: RT_QG(8); break;
  }
#undef RT_QG
  RT_LAUNCH_CHECK();
}

void q_gemv(const QGemvArgs& a, cudaStream_t stream) {
  RT_CHECK(a.K % 32 == 0, "q_gemv: K must be a multiple of 32");
  RT_CHECK(a.ldx % 8 == 0, "q_gemv: activation row stride must be a multiple of 8 halves");
  RT_CHECK((reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.qs) & 15) == 0,
           "q_gemv: x and qs must be 16-byte aligned");
  if (a.M == 0 || a.N == 0) return;
  for (int m0 = 0; m0 < a.M; m0 += 8) {
    const int m = std::min(8, a.M - m0);
    if (a.q8) launch_rows<true>(a, m0, m, stream);
    else launch_rows<false>(a, m0, m, stream);
  }
}

// ---------------------------------------------------------------------------- repack
// GGUF Q4_0 block stream [rows][K/32][18] -> qs (uint4 per block, layout above) + scales.
__global__ void repack_q4_0_kernel(const uint8_t* __restrict__ blocks, uint4* __restrict__ qs,
                                   __half* __restrict__ scales, long long n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  const uint8_t* b = blocks + i * 18;
  scales[i] = __ushort_as_half((unsigned short)(b[0] | (b[1] << 8)));
  uint32_t out[4];
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int k = wi * 8 + e;  // weight index in the block
      const uint32_t q = (k < 16) ? (b[2 + k] & 0x0F) : (b[2 + k - 16] >> 4);
      const int shift = (e & 1) ? 16 + 4 * (e >> 1) : 4 * (e >> 1);
      word |= q << shift;
    }
    out[wi] = word;
  }
  qs[i] = make_uint4(out[0], out[1], out[2], out[3]);
}

// GGUF Q8_0 block stream [rows][K/32][34] -> qs int8 [.][32] + scales.
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ blocks, int8_t* __restrict__ qs,
                                   __half* __restrict__ scales, long long n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  const uint8_t* b = blocks + i * 34;
  scales[i] = __ushort_as_half((unsigned short)(b[0] | (b[1] << 8)));
  for (int k = 0; k < 32; ++k) qs[i * 32 + k] = (int8_t)b[2 + k];
}

void repack_q4_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s) {
  if (n_blocks == 0) return;
  repack_q4_0_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const uint8_t*>(blocks), reinterpret_cast<uint4*>(qs), reinterpret_cast<__half*>(scales), n_blocks);
  RT_LAUNCH_CHECK();
}

void repack_q8_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s) {
  if (n_blocks == 0) return;
  repack_q8_0_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const uint8_t*>(blocks), reinterpret_cast<int8_t*>(qs), reinterpret_cast<__half*>(scales), n_blocks);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
