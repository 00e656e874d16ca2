// GroupNorm and InstanceNorm (= GroupNorm with one channel per group) over a contiguous [N][C][HW] tensor,
// bf16 / fp16 / fp32 storage, fp32 statistics.  One CTA owns one (sample, group) slab, which is contiguous
// ((C/G) * HW elements), so both passes of a direction stream one slab: the second pass finds it in L1/L2.
//
//   forward   mean / rstd over the slab, y = (x - mean) * rstd * gamma[c] + beta[c]; mean and rstd saved [N*G]
//   backward  per channel a_c = sum(dy), b_c = sum(dy * xhat) (one atomic per channel into dbeta / dgamma),
//             s1 = sum_c gamma_c a_c, s2 = sum_c gamma_c b_c, dx = rstd * (dy gamma_c - s1/L - xhat s2/L)
//
// The reference normalises with scalar host loops over Vec<f32> (src/nn/normalization.rs:343-520 GroupNorm,
// src/nn/instance_norm.rs:148-330 InstanceNorm1d/2d/3d) and has no device kernel for either.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

constexpr int GN_THREADS = 512;

template <typename T> struct GnVec { static constexpr int N = 8; };
template <> struct GnVec<float> { static constexpr int N = 4; };

__device__ __forceinline__ float gn_tf(float v) { return v; }
__device__ __forceinline__ float gn_tf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float gn_tf(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T gn_ff(float v);
template <> __device__ __forceinline__ float gn_ff<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gn_ff<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half gn_ff<__half>(float v) { return __float2half(v); }

template <typename T>
__device__ __forceinline__ void gn_ld(const T* p, float (&f)[GnVec<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < GnVec<T>::N; ++i) f[i] = gn_tf(e[i]);
}
template <typename T>
__device__ __forceinline__ void gn_st(T* p, const float (&f)[GnVec<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < GnVec<T>::N; ++i) e[i] = gn_ff<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Sum of (a, b) over the CTA; every thread gets the result.  red: 2 * 32 floats of shared memory.
__device__ __forceinline__ void gn_block_sum2(float& a, float& b, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();  // red may still be read from an earlier call
  if (lane == 0) {
    red[warp] = a;
    red[32 + warp] = b;
  }
  __syncthreads();
  a = lane < nw ? red[lane] : 0.f;
  b = lane < nw ? red[32 + lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
}

// VEC: HW is a multiple of the vector width and the tensor is 16-byte aligned, so a vector never straddles channels.
template <typename T, bool VEC>
__global__ void __launch_bounds__(GN_THREADS) gn_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                            const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            float* __restrict__ mean, float* __restrict__ rstd, int C, int G,
                                                            long long HW, float eps) {
  constexpr int V = VEC ? GnVec<T>::N : 1;
  __shared__ float red[64];
  const int cpg = C / G;
  const long long L = (long long)cpg * HW;
  const long long slab = blockIdx.x;  // n * G + g
  const int g = (int)(slab % G);
  const T* xs = x + slab * L;
  T* ys = y + slab * L;
  float a = 0.f, b = 0.f;
  for (long long i = (long long)threadIdx.x * V; i < L; i += (long long)blockDim.x * V) {
    if (VEC) {
      float f[GnVec<T>::N];
      gn_ld(xs + i, f);
#pragma unroll
      for (int e = 0; e < GnVec<T>::N; ++e) {
        a += f[e];
        b = fmaf(f[e], f[e], b);
      }
    } else {
      const float f = gn_tf(xs[i]);
      a += f;
      b = fmaf(f, f, b);
    }
  }
  gn_block_sum2(a, b, red);
  const float mu = a / (float)L;
  const float rs = rsqrtf(fmaxf(b / (float)L - mu * mu, 0.f) + eps);
  if (threadIdx.x == 0) {
    mean[slab] = mu;
    rstd[slab] = rs;
  }
  for (long long i = (long long)threadIdx.x * V; i < L; i += (long long)blockDim.x * V) {
    const int c = g * cpg + (int)(i / HW);
    const float sc = rs * (gamma ? gamma[c] : 1.f);
    const float sh = (beta ? beta[c] : 0.f) - mu * sc;
    if (VEC) {
      float f[GnVec<T>::N];
      gn_ld(xs + i, f);
#pragma unroll
      for (int e = 0; e < GnVec<T>::N; ++e) f[e] = fmaf(f[e], sc, sh);
      gn_st(ys + i, f);
    } else {
      ys[i] = gn_ff<T>(fmaf(gn_tf(xs[i]), sc, sh));
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(GN_THREADS) gn_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                                                            const float* __restrict__ gamma, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, float* __restrict__ dgamma,
                                                            float* __restrict__ dbeta, int C, int G, long long HW) {
  constexpr int V = VEC ? GnVec<T>::N : 1;
  __shared__ float red[64];
  const int cpg = C / G;
  const long long L = (long long)cpg * HW;
  const long long slab = blockIdx.x;
  const int g = (int)(slab % G);
  const T* xs = x + slab * L;
  const T* gs = dy + slab * L;
  T* ds = dx + slab * L;
  const float mu = mean[slab], rs = rstd[slab];
  float s1 = 0.f, s2 = 0.f;
  for (int cl = 0; cl < cpg; ++cl) {
    const int c = g * cpg + cl;
    const T* xc = xs + (long long)cl * HW;
    const T* gc = gs + (long long)cl * HW;
    float a = 0.f, b = 0.f;
    for (long long i = (long long)threadIdx.x * V; i < HW; i += (long long)blockDim.x * V) {
      if (VEC) {
        float fx[GnVec<T>::N], fg[GnVec<T>::N];
        gn_ld(xc + i, fx);
        gn_ld(gc + i, fg);
#pragma unroll
        for (int e = 0; e < GnVec<T>::N; ++e) {
          a += fg[e];
          b = fmaf(fg[e], (fx[e] - mu) * rs, b);
        }
      } else {
        const float fg = gn_tf(gc[i]);
        a += fg;
        b = fmaf(fg, (gn_tf(xc[i]) - mu) * rs, b);
      }
    }
    gn_block_sum2(a, b, red);
    if (threadIdx.x == 0) {
      if (dbeta) atomicAdd(dbeta + c, a);
      if (dgamma) atomicAdd(dgamma + c, b);
    }
    const float gm = gamma ? gamma[c] : 1.f;
    s1 = fmaf(gm, a, s1);
    s2 = fmaf(gm, b, s2);
  }
  const float k1 = s1 / (float)L, k2 = s2 / (float)L;
  for (long long i = (long long)threadIdx.x * V; i < L; i += (long long)blockDim.x * V) {
    const int c = g * cpg + (int)(i / HW);
    const float gm = gamma ? gamma[c] : 1.f;
    if (VEC) {
      float fx[GnVec<T>::N], fg[GnVec<T>::N];
      gn_ld(xs + i, fx);
      gn_ld(gs + i, fg);
#pragma unroll
      for (int e = 0; e < GnVec<T>::N; ++e) fx[e] = rs * (fg[e] * gm - k1 - (fx[e] - mu) * rs * k2);
      gn_st(ds + i, fx);
    } else {
      ds[i] = gn_ff<T>(rs * (gn_tf(gs[i]) * gm - k1 - (gn_tf(xs[i]) - mu) * rs * k2));
    }
  }
}

template <typename T>
void gn_launch(const GroupNormArgs& a, bool bwd, cudaStream_t s) {
  constexpr int V = GnVec<T>::N;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = a.HW % V == 0 && aligned(a.x) && (bwd ? aligned(a.dy) && aligned(a.dx) : aligned(a.y));
  const unsigned grid = (unsigned)(a.N * a.G);
  auto px = reinterpret_cast<const T*>(a.x);
  if (!bwd) {
    auto kern = vec ? gn_fwd_kernel<T, true> : gn_fwd_kernel<T, false>;
    kern<<<grid, GN_THREADS, 0, s>>>(px, reinterpret_cast<T*>(a.y), a.gamma, a.beta, a.mean, a.rstd, a.C, a.G, a.HW, a.eps);
  } else {
    auto kern = vec ? gn_bwd_kernel<T, true> : gn_bwd_kernel<T, false>;
    kern<<<grid, GN_THREADS, 0, s>>>(px, reinterpret_cast<const T*>(a.dy), reinterpret_cast<T*>(a.dx), a.gamma, a.mean, a.rstd,
                                     a.dgamma, a.dbeta, a.C, a.G, a.HW);
  }
  RT_LAUNCH_CHECK();
}

void gn_check(const GroupNormArgs& a) {
  RT_CHECK(a.dtype >= DT_F32 && a.dtype <= DT_F16, "groupnorm: dtype must be fp32, bf16 or fp16");
  RT_CHECK(a.N > 0 && a.C > 0 && a.G > 0 && a.HW > 0 && a.C % a.G == 0, "groupnorm: channels must divide into the groups");
  RT_CHECK(a.N * a.G < (1LL << 31), "groupnorm: too many (sample, group) slabs for one grid");
  RT_CHECK(a.x && a.mean && a.rstd, "groupnorm: missing buffers");
}

}  // namespace

void groupnorm_fwd(const GroupNormArgs& a, cudaStream_t s) {
  gn_check(a);
  RT_CHECK(a.y != nullptr, "groupnorm_fwd: y required");
  if (a.dtype == DT_F32) gn_launch<float>(a, false, s);
  else if (a.dtype == DT_BF16) gn_launch<__nv_bfloat16>(a, false, s);
  else gn_launch<__half>(a, false, s);
}

// dgamma / dbeta (fp32 [C], may be null) are accumulated into: the caller zeroes them.
void groupnorm_bwd(const GroupNormArgs& a, cudaStream_t s) {
  gn_check(a);
  RT_CHECK(a.dy && a.dx, "groupnorm_bwd: dy and dx required");
  if (a.dtype == DT_F32) gn_launch<float>(a, true, s);
  else if (a.dtype == DT_BF16) gn_launch<__nv_bfloat16>(a, true, s);
  else gn_launch<__half>(a, true, s);
}

}  // namespace rt
