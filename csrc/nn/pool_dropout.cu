// Pooling over channels-last activations and counter-based dropout, forward and backward, fp32 / bf16 / fp16.
//
//   max_pool2d   out[n][oh][ow][c] = max over the kh x kw window (padding reads as -inf); the window position of the
//                maximum (first one in scan order, as PyTorch) is kept as one byte per output element, so that the
//                backward pass is a gather: every input pixel sums the gradients of the <= ceil(k/s)^2 outputs whose
//                recorded maximum is that pixel.  No atomics, no index tensor of 8-byte integers.
//   avg_pool2d   mean over the window, padding counted in the divisor (count_include_pad, the PyTorch default);
//                adaptive pooling to 1 x 1 is the same kernel with the window equal to the image.
//   dropout      y = x * keep / (1 - p) with keep drawn from Philox4x32-10 keyed by (seed, offset) and counted by
//                element index / 4; the backward pass regenerates the same bits from (seed, offset), so no mask is
//                stored or read (the reference materialises a mask tensor, src/nn/dropout.rs:105-176).
//
// A thread owns 16 bytes of channels (8 x 16-bit or 4 x 32-bit) of one output pixel; C must be a multiple of that.
// Reference: src/nn/pool2d.rs:34-330 (NCHW scalar loops), src/nn/adaptive_pool.rs:47-260.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cfloat>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

template <typename T> struct PVec { static constexpr int N = 8; };
template <> struct PVec<float> { static constexpr int N = 4; };
__device__ __forceinline__ float pf(float v) { return v; }
__device__ __forceinline__ float pf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float pf(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T pt(float v);
template <> __device__ __forceinline__ float pt<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 pt<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half pt<__half>(float v) { return __float2half(v); }

template <typename T>
__device__ __forceinline__ void pload(const T* p, float (&f)[PVec<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < PVec<T>::N; ++i) f[i] = pf(e[i]);
}
template <typename T>
__device__ __forceinline__ void punpack(const uint4& raw, float (&f)[PVec<T>::N]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < PVec<T>::N; ++i) f[i] = pf(e[i]);
}
template <typename T>
__device__ __forceinline__ void pstore(T* p, const float (&f)[PVec<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < PVec<T>::N; ++i) e[i] = pt<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ------------------------------------------------------------------------------------------------ pooling
// K, S: square window and stride known at compile time (0 = read them from the arguments).  With constants the tap
// loops unroll, so all window loads of a thread are in flight together and the index arithmetic has no divisions
// by runtime strides.
template <typename T, bool MAX, int K, int S>
__global__ void __launch_bounds__(256, 3) pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, unsigned char* __restrict__ idx,
                                                       const Pool2dArgs a) {
  constexpr int V = PVec<T>::N;
  const int cv = a.C / V;
  const int KH = K ? K : a.kh, KW = K ? K : a.kw, SH = S ? S : a.sh, SW = S ? S : a.sw;
  const long long total = (long long)a.N * a.OH * a.OW * cv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c, ow, oh, n;
    if (total < 0x7fffffffLL) {
      const unsigned tt = (unsigned)t, pix = tt / (unsigned)cv, row = pix / (unsigned)a.OW;
      c = (int)(tt - pix * cv) * V;
      ow = (int)(pix - row * a.OW);
      n = (int)(row / (unsigned)a.OH);
      oh = (int)(row - (unsigned)n * a.OH);
    } else {
      c = (int)(t % cv) * V;
      long long pix = t / cv;
      ow = (int)(pix % a.OW);
      pix /= a.OW;
      oh = (int)(pix % a.OH);
      n = (int)(pix / a.OH);
    }
    float acc[V];
    __align__(8) unsigned char best[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = MAX ? -INFINITY : 0.f, best[i] = 0;
    const int h0 = oh * SH - a.ph, w0 = ow * SW - a.pw;
    const T* xn = x + (long long)n * a.H * a.W * a.C + c;
    if (K) {
      // all taps loaded first (out-of-image taps are skipped by predicate), then reduced in tap order
      uint4 v[(K ? K * K : 1)];      // raw vectors: 4 registers per tap while the loads are in flight
      bool in[(K ? K * K : 1)];
#pragma unroll
      for (int kh = 0; kh < K; ++kh)
#pragma unroll
        for (int kw = 0; kw < K; ++kw) {
          const int ih = h0 + kh, iw = w0 + kw;
          in[kh * K + kw] = ih >= 0 && ih < a.H && iw >= 0 && iw < a.W;
          if (in[kh * K + kw]) v[kh * K + kw] = *reinterpret_cast<const uint4*>(xn + ((long long)ih * a.W + iw) * a.C);
        }
#pragma unroll
      for (int tap = 0; tap < K * K; ++tap) {
        if (!in[tap]) continue;
        float f[V];
        punpack<T>(v[tap], f);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if (MAX) {
            if (f[i] > acc[i] || f[i] != f[i]) acc[i] = f[i], best[i] = (unsigned char)tap;
          } else {
            acc[i] += f[i];
          }
        }
      }
    } else {
      for (int kh = 0; kh < KH; ++kh) {
        const int ih = h0 + kh;
        if (ih < 0 || ih >= a.H) continue;
        for (int kw = 0; kw < KW; ++kw) {
          const int iw = w0 + kw;
          if (iw < 0 || iw >= a.W) continue;
          float v[V];
          pload(xn + ((long long)ih * a.W + iw) * a.C, v);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            if (MAX) {
              if (v[i] > acc[i] || v[i] != v[i]) acc[i] = v[i], best[i] = (unsigned char)(kh * KW + kw);
            } else {
              acc[i] += v[i];
            }
          }
        }
      }
    }
    if (!MAX) {
      const float inv = 1.f / (float)(KH * KW);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] *= inv;
    }
    const long long o = (((long long)n * a.OH + oh) * a.OW + ow) * a.C + c;
    pstore(y + o, acc);
    if (MAX && idx != nullptr) {
      if (V == 8) *reinterpret_cast<uint2*>(idx + o) = *reinterpret_cast<const uint2*>(best);
      else *reinterpret_cast<unsigned*>(idx + o) = *reinterpret_cast<const unsigned*>(best);
    }
  }
}

template <typename T, bool MAX, int K, int S>
__global__ void __launch_bounds__(256) pool_bwd_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx,
                                                       T* __restrict__ dx, const Pool2dArgs a) {
  constexpr int V = PVec<T>::N;
  const int cv = a.C / V;
  const int KH = K ? K : a.kh, KW = K ? K : a.kw, SH = S ? S : a.sh, SW = S ? S : a.sw;
  const long long total = (long long)a.N * a.H * a.W * cv;
  const float inv = 1.f / (float)(KH * KW);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c, iw, ih, n;
    if (total < 0x7fffffffLL) {                      // 32-bit divisions (an order of magnitude cheaper than 64-bit ones)
      const unsigned tt = (unsigned)t, pix = tt / (unsigned)cv, row = pix / (unsigned)a.W;
      c = (int)(tt - pix * cv) * V;
      iw = (int)(pix - row * a.W);
      n = (int)(row / (unsigned)a.H);
      ih = (int)(row - (unsigned)n * a.H);
    } else {
      c = (int)(t % cv) * V;
      long long pix = t / cv;
      iw = (int)(pix % a.W);
      pix /= a.W;
      ih = (int)(pix % a.H);
      n = (int)(pix / a.H);
    }
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    // outputs whose window contains (ih, iw): oh in [ceil((ih + ph - kh + 1) / sh), floor((ih + ph) / sh)]
    const int oh_top = (ih + a.ph) / SH, ow_top = (iw + a.pw) / SW;
    const T* gn = dy + (long long)n * a.OH * a.OW * a.C + c;
    const unsigned char* in_ = idx ? idx + (long long)n * a.OH * a.OW * a.C + c : nullptr;
    if (K) {
      constexpr int NC = K ? (K + (S ? S : 1) - 1) / (S ? S : 1) : 1;   // candidate outputs per direction
      uint4 g[NC * NC];
      __align__(8) unsigned char rec[NC * NC][8];
      bool in[NC * NC];
      unsigned char me[NC * NC];
#pragma unroll
      for (int jh = 0; jh < NC; ++jh)
#pragma unroll
        for (int jw = 0; jw < NC; ++jw) {
          const int q = jh * NC + jw;
          const int oh = oh_top - jh, ow = ow_top - jw;
          const int kh = ih + a.ph - oh * SH, kw = iw + a.pw - ow * SW;     // >= 0 by construction
          in[q] = oh >= 0 && oh < a.OH && ow >= 0 && ow < a.OW && kh < K && kw < K;
          me[q] = (unsigned char)(kh * K + kw);
          if (in[q]) {
            const long long o = ((long long)oh * a.OW + ow) * a.C;
            g[q] = *reinterpret_cast<const uint4*>(gn + o);
            if (MAX) {
              if (V == 8) *reinterpret_cast<uint2*>(rec[q]) = *reinterpret_cast<const uint2*>(in_ + o);
              else *reinterpret_cast<unsigned*>(rec[q]) = *reinterpret_cast<const unsigned*>(in_ + o);
            }
          }
        }
#pragma unroll
      for (int q = NC * NC - 1; q >= 0; --q) {     // ascending (oh, ow), the order of the runtime path
        if (!in[q]) continue;
        float f[V];
        punpack<T>(g[q], f);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if (MAX) {
            if (rec[q][i] == me[q]) acc[i] += f[i];
          } else {
            acc[i] += f[i] * inv;
          }
        }
      }
    } else {
      const int oh_hi = min(a.OH - 1, oh_top), ow_hi = min(a.OW - 1, ow_top);
      const int oh_lo = max(0, (ih + a.ph - KH + SH) / SH), ow_lo = max(0, (iw + a.pw - KW + SW) / SW);
      for (int oh = oh_lo; oh <= oh_hi; ++oh) {
        const int kh = ih + a.ph - oh * SH;
        if (kh < 0 || kh >= KH) continue;
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
          const int kw = iw + a.pw - ow * SW;
          if (kw < 0 || kw >= KW) continue;
          const long long o = ((long long)oh * a.OW + ow) * a.C;
          float g[V];
          pload(gn + o, g);
          if (MAX) {
            const unsigned char me = (unsigned char)(kh * KW + kw);
            __align__(8) unsigned char rec[V];         // V consecutive bytes: one 4- or 8-byte load
            if (V == 8) *reinterpret_cast<uint2*>(rec) = *reinterpret_cast<const uint2*>(in_ + o);
            else *reinterpret_cast<unsigned*>(rec) = *reinterpret_cast<const unsigned*>(in_ + o);
#pragma unroll
            for (int i = 0; i < V; ++i)
              if (rec[i] == me) acc[i] += g[i];
          } else {
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += g[i] * inv;
          }
        }
      }
    }
    pstore(dx + (((long long)n * a.H + ih) * a.W + iw) * a.C + c, acc);
  }
}

// ------------------------------------------------------------------------------------------------ dropout
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const unsigned hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// One Philox call covers 4 consecutive elements; a thread handles one 16-byte vector (1 or 2 calls).
template <typename T>
__global__ void __launch_bounds__(256) dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p, float scale,
                                                      unsigned long long seed, unsigned long long offset) {
  constexpr int V = PVec<T>::N;
  const long long nvec = n / V;
  const unsigned thresh = (unsigned)fmin(4294967295.0, (double)p * 4294967296.0);   // drop when bits < thresh
  const uint2 key = make_uint2((unsigned)seed, (unsigned)(seed >> 32));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float v[V];
    pload(x + i * V, v);
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const unsigned long long cnt = (unsigned long long)(i * (V / 4) + q);
      const uint4 r = philox4x32_10(make_uint4((unsigned)cnt, (unsigned)(cnt >> 32), (unsigned)offset, (unsigned)(offset >> 32)), key);
      const unsigned bits[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) v[q * 4 + e] = bits[e] < thresh ? 0.f : v[q * 4 + e] * scale;
    }
    pstore(y + i * V, v);
  }
}

int grid_for(long long work, int device) { return (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, 8LL * sm_count(device))); }

}  // namespace

void pool2d(const Pool2dArgs& a, cudaStream_t stream) {
  RT_CHECK(a.dtype >= DT_F32 && a.dtype <= DT_F16, "pool2d: dtype must be fp32, bf16 or fp16");
  const int V = a.dtype == DT_F32 ? 4 : 8;
  RT_CHECK(a.C % V == 0, "pool2d: channel count must be a multiple of the 16-byte vector");
  RT_CHECK(a.kh >= 1 && a.kw >= 1 && a.kh * a.kw <= 255 && a.sh >= 1 && a.sw >= 1 && a.ph >= 0 && a.pw >= 0, "pool2d: bad window");
  RT_CHECK(a.OH == (a.H + 2 * a.ph - a.kh) / a.sh + 1 && a.OW == (a.W + 2 * a.pw - a.kw) / a.sw + 1, "pool2d: output size mismatch");
  RT_CHECK(!a.backward || !a.max || a.idx != nullptr, "pool2d: max-pool backward needs the recorded window positions");
  const int device = current_device();
  const long long work = (long long)a.N * (a.backward ? (long long)a.H * a.W : (long long)a.OH * a.OW) * (a.C / V);
  if (work == 0) return;
  const int grid = grid_for(work, device);
#define RT_POOL(T, K, S)                                                                                                              \
  do {                                                                                                                          \
    if (!a.backward) {                                                                                                          \
      if (a.max) pool_fwd_kernel<T, true, K, S><<<grid, 256, 0, stream>>>((const T*)a.x, (T*)a.y, a.idx, a);                    \
      else pool_fwd_kernel<T, false, K, S><<<grid, 256, 0, stream>>>((const T*)a.x, (T*)a.y, nullptr, a);                       \
    } else {                                                                                                                    \
      if (a.max) pool_bwd_kernel<T, true, K, S><<<grid, 256, 0, stream>>>((const T*)a.y, a.idx, (T*)a.x, a);                    \
      else pool_bwd_kernel<T, false, K, S><<<grid, 256, 0, stream>>>((const T*)a.y, nullptr, (T*)a.x, a);                       \
    }                                                                                                                           \
  } while (0)
#define RT_POOL_T(K, S)                                                                                                         \
  do {                                                                                                                          \
    if (a.dtype == DT_F32) RT_POOL(float, K, S);                                                                                \
    else if (a.dtype == DT_BF16) RT_POOL(__nv_bfloat16, K, S);                                                                  \
    else RT_POOL(__half, K, S);                                                                                                 \
  } while (0)
  const bool square = a.kh == a.kw && a.sh == a.sw;
  if (square && a.kh == 3 && a.sh == 2) RT_POOL_T(3, 2);
  else if (square && a.kh == 2 && a.sh == 2) RT_POOL_T(2, 2);
  else RT_POOL_T(0, 0);
#undef RT_POOL_T
#undef RT_POOL
  RT_LAUNCH_CHECK();
}

void dropout(int dtype, const void* x, void* y, long long n, float p, unsigned long long seed, unsigned long long offset,
             cudaStream_t stream) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "dropout: dtype must be fp32, bf16 or fp16");
  RT_CHECK(p >= 0.f && p < 1.f, "dropout: p must be in [0, 1)");
  const int V = dtype == DT_F32 ? 4 : 8;
  RT_CHECK(n % V == 0, "dropout: element count must be a multiple of the 16-byte vector");
  if (n == 0) return;
  const int grid = grid_for(n / V, current_device());
  const float scale = 1.f / (1.f - p);
  if (dtype == DT_F32) dropout_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)y, n, p, scale, seed, offset);
  else if (dtype == DT_BF16)
    dropout_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p, scale, seed, offset);
  else dropout_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)x, (__half*)y, n, p, scale, seed, offset);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
