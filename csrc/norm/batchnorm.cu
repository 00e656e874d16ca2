// BatchNorm (1d / 2d / 3d) training and inference kernels over a channels-last matrix x[M][C]
// (M = N*H*W pixels, C channels contiguous), bf16 / fp16 / fp32 storage, fp32 statistics.
//
// The reference computes batch statistics with scalar host loops (src/nn/batchnorm.rs:120-330) and
// ships a CUDA-C "batch_norm" string kernel that only applies precomputed statistics (K6,
// src/gpu/cuda_kernels.rs:332-372).  Here:
//   bn_stats      per-channel sum and sum of squares: each CTA walks a slab of rows with 16-byte loads,
//                 threads own a group of 8 (4 for fp32) channels, rows are split over the thread rows of the
//                 CTA, partials meet in shared memory and one float atomic per channel per CTA lands in
//                 global memory;
//   bn_apply      y = (x - mean) * rstd * gamma + beta, optionally + residual and ReLU (the ResNet block
//                 tail), and CTA 0 updates running_mean / running_var (unbiased) with the momentum;
//   bn_bwd_reduce per-channel sum(dy) and sum(dy * xhat), dy masked by the fused ReLU where present;
//   bn_bwd_apply  dx = gamma * rstd * (dy - sum_dy / M - xhat * sum_dy_xhat / M)  (and the residual grad).
// Every pass is a single stream over x (or x and dy): HBM-bound, two passes forward, two backward.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

template <typename T> struct VecN { static constexpr int N = 8; };
template <> struct VecN<float> { static constexpr int N = 4; };

__device__ __forceinline__ float tf(float v) { return v; }
__device__ __forceinline__ float tf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float tf(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T ff(float v);
template <> __device__ __forceinline__ float ff<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 ff<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half ff<__half>(float v) { return __float2half(v); }

template <typename T>
__device__ __forceinline__ void ldv(const T* p, float (&f)[VecN<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < VecN<T>::N; ++i) f[i] = tf(e[i]);
}
template <typename T>
__device__ __forceinline__ void stv(T* p, const float (&f)[VecN<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < VecN<T>::N; ++i) e[i] = ff<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// CTA shape for every kernel here: blockDim.x = channel groups handled side by side (a power of two <= 32),
// blockDim.y = row lanes.  A thread keeps one channel group for its whole life, so the per-channel constants sit
// in registers, and it walks rows r = first + k * row_step with U independent 16-byte loads in flight.
// Two accumulators per channel (A, B): forward (x, x^2); backward (dy, dy * xhat).
template <typename T, bool BWD>
__global__ void __launch_bounds__(512) bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const T* __restrict__ y_relu, const float* __restrict__ mean,
                                                        const float* __restrict__ rstd, float* __restrict__ out,
                                                        long long M, int C, long long rows_per_cta) {
  constexpr int V = VecN<T>::N;
  constexpr int U = BWD ? 2 : 4;
  extern __shared__ float sm[];  // [2][blockDim.y][blockDim.x * V]
  const int cgroups = C / V;
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * rows_per_cta;
  const long long r1 = min(M, r0 + rows_per_cta);
  const long long step = blockDim.y;
  float a[V], b[V];
#pragma unroll
  for (int i = 0; i < V; ++i) a[i] = b[i] = 0.f;
  if (cg < cgroups) {
    float mu[V], rs[V];
    if (BWD) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        mu[i] = mean[cg * V + i];
        rs[i] = rstd[cg * V + i];
      }
    }
    auto accumulate = [&](const float (&xv)[V], float (&g)[V], const float (&yv)[V], bool masked) {
      if (!BWD) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          a[i] += xv[i];
          b[i] = fmaf(xv[i], xv[i], b[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float gi = (masked && !(yv[i] > 0.f)) ? 0.f : g[i];
          a[i] += gi;
          b[i] = fmaf(gi, (xv[i] - mu[i]) * rs[i], b[i]);
        }
      }
    };
    const size_t col = (size_t)cg * V;
    long long r = r0 + threadIdx.y;
    for (; r + (U - 1) * step < r1; r += U * step) {
      float xv[U][V], g[U][V], yv[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t off = (size_t)(r + u * step) * C + col;
        ldv(x + off, xv[u]);
        if (BWD) {
          ldv(dy + off, g[u]);
          if (y_relu) ldv(y_relu + off, yv[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) accumulate(xv[u], g[u], yv[u], y_relu != nullptr);
    }
    for (; r < r1; r += step) {
      float xv[V], g[V], yv[V];
      const size_t off = (size_t)r * C + col;
      ldv(x + off, xv);
      if (BWD) {
        ldv(dy + off, g);
        if (y_relu) ldv(y_relu + off, yv);
      }
      accumulate(xv, g, yv, y_relu != nullptr);
    }
  }
  const int W = blockDim.x * V;
  float* sa = sm + (size_t)threadIdx.y * W + threadIdx.x * V;
  float* sb = sa + (size_t)blockDim.y * W;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    sa[i] = a[i];
    sb[i] = b[i];
  }
  __syncthreads();
  // column sums over the row lanes: thread t handles column t (and t + nthreads ...)
  const int nth = blockDim.x * blockDim.y, tid = threadIdx.y * blockDim.x + threadIdx.x;
  for (int col = tid; col < 2 * W; col += nth) {
    const int which = col / W, c = col % W;
    const int ch = blockIdx.x * W + c;
    if (ch >= C) continue;
    float s = 0.f;
    for (int ry = 0; ry < (int)blockDim.y; ++ry) s += sm[((size_t)which * blockDim.y + ry) * W + c];
    atomicAdd(out + (size_t)which * C + ch, s);
  }
}

// Forward apply.  stats = [2][C] sums from bn_reduce (training) or null (inference: uses running stats).
// y = x * scale + shift per channel (+ residual, ReLU); the CTAs of grid row 0 write the saved and running statistics.
template <typename T>
__global__ void __launch_bounds__(256) bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ residual, T* __restrict__ y,
                                                       const float* __restrict__ stats, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, float* __restrict__ running_mean,
                                                       float* __restrict__ running_var, float* __restrict__ save_mean,
                                                       float* __restrict__ save_rstd, long long M, int C, float eps,
                                                       float momentum, int relu, int training) {
  constexpr int V = VecN<T>::N;
  constexpr int U = 4;
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;
  if (cg >= C / V) return;
  const float invM = 1.f / (float)M;
  float scale[V], shift[V];
  const bool writer = training && blockIdx.y == 0 && threadIdx.y == 0;
#pragma unroll
  for (int e = 0; e < V; ++e) {
    const int c = cg * V + e;
    float mu, var;
    if (training) {
      mu = stats[c] * invM;
      var = fmaxf(stats[C + c] * invM - mu * mu, 0.f);
    } else {
      mu = running_mean[c];
      var = running_var[c];
    }
    const float rs = rsqrtf(var + eps);
    scale[e] = rs * (gamma ? gamma[c] : 1.f);
    shift[e] = (beta ? beta[c] : 0.f) - mu * scale[e];
    if (writer) {
      if (save_mean) save_mean[c] = mu;
      if (save_rstd) save_rstd[c] = rs;
      if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
      if (running_var) {
        const float unbiased = M > 1 ? var * (float)M / (float)(M - 1) : var;
        running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
      }
    }
  }
  const size_t col = (size_t)cg * V;
  const long long step = (long long)gridDim.y * blockDim.y;
  auto finish = [&](float (&o)[V], const float (&rv)[V]) {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      o[e] = fmaf(o[e], scale[e], shift[e]);
      if (residual) o[e] += rv[e];
      if (relu) o[e] = fmaxf(o[e], 0.f);
    }
  };
  long long r = (long long)blockIdx.y * blockDim.y + threadIdx.y;
  for (; r + (U - 1) * step < M; r += U * step) {
    float o[U][V], rv[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t off = (size_t)(r + u * step) * C + col;
      ldv(x + off, o[u]);
      if (residual) ldv(residual + off, rv[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      finish(o[u], rv[u]);
      stv(y + (size_t)(r + u * step) * C + col, o[u]);
    }
  }
  for (; r < M; r += step) {
    float o[V], rv[V];
    const size_t off = (size_t)r * C + col;
    ldv(x + off, o);
    if (residual) ldv(residual + off, rv);
    finish(o, rv);
    stv(y + off, o);
  }
}

// dx (and the residual branch gradient = masked dy) from the per-channel sums in `sums` = [2][C]:
// dx = ka * dy + kb * x + kc with ka = gamma * rstd, kb = -ka * rstd * sum(dy xhat) / M, kc = -ka * sum(dy) / M - kb * mean.
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                           const T* __restrict__ y_relu, T* __restrict__ dx,
                                                           T* __restrict__ dres, const float* __restrict__ sums,
                                                           const float* __restrict__ mean, const float* __restrict__ rstd,
                                                           const float* __restrict__ gamma, long long M, int C) {
  constexpr int V = VecN<T>::N;
  constexpr int U = 2;
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;
  if (cg >= C / V) return;
  const float invM = 1.f / (float)M;
  float ka[V], kb[V], kc[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    const int c = cg * V + e;
    ka[e] = (gamma ? gamma[c] : 1.f) * rstd[c];
    kb[e] = -ka[e] * rstd[c] * sums[C + c] * invM;
    kc[e] = -ka[e] * sums[c] * invM - kb[e] * mean[c];
  }
  const size_t col = (size_t)cg * V;
  const long long step = (long long)gridDim.y * blockDim.y;
  auto finish = [&](const float (&xv)[V], float (&g)[V], const float (&yv)[V], float (&o)[V]) {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (y_relu && !(yv[e] > 0.f)) g[e] = 0.f;
      o[e] = fmaf(ka[e], g[e], fmaf(kb[e], xv[e], kc[e]));
    }
  };
  long long r = (long long)blockIdx.y * blockDim.y + threadIdx.y;
  for (; r + (U - 1) * step < M; r += U * step) {
    float xv[U][V], g[U][V], yv[U][V], o[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t off = (size_t)(r + u * step) * C + col;
      ldv(x + off, xv[u]);
      ldv(dy + off, g[u]);
      if (y_relu) ldv(y_relu + off, yv[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t off = (size_t)(r + u * step) * C + col;
      finish(xv[u], g[u], yv[u], o[u]);
      stv(dx + off, o[u]);
      if (dres) stv(dres + off, g[u]);
    }
  }
  for (; r < M; r += step) {
    float xv[V], g[V], yv[V], o[V];
    const size_t off = (size_t)r * C + col;
    ldv(x + off, xv);
    ldv(dy + off, g);
    if (y_relu) ldv(y_relu + off, yv);
    finish(xv, g, yv, o);
    stv(dx + off, o);
    if (dres) stv(dres + off, g);
  }
}

// Channel groups side by side (a power of two <= 32) and the CTA grid for `threads` threads per CTA.
struct BnShape {
  dim3 grid, block;
};
BnShape bn_shape(long long M, int cgroups, int threads, int unroll, int ctas_per_sm) {
  int bx = 1;
  while (bx < cgroups && bx < 32) bx <<= 1;
  const int by = threads / bx;
  const int gx = (cgroups + bx - 1) / bx;
  const long long want = ((long long)sm_count(current_device()) * ctas_per_sm + gx - 1) / gx;
  const long long gy = std::max<long long>(1, std::min<long long>((M + (long long)by * unroll - 1) / ((long long)by * unroll), want));
  return {dim3(gx, (unsigned)gy), dim3(bx, by)};
}

template <typename T>
void launch_reduce(const BatchNormArgs& a, bool bwd, float* out, cudaStream_t s) {
  constexpr int V = VecN<T>::N;
  BnShape sh = bn_shape(a.M, a.C / V, 512, 4, 4);
  const long long rows_per_cta = (a.M + sh.grid.y - 1) / sh.grid.y;
  sh.grid.y = (unsigned)((a.M + rows_per_cta - 1) / rows_per_cta);
  const size_t smem = sizeof(float) * 2 * sh.block.y * sh.block.x * V;
  auto px = reinterpret_cast<const T*>(a.x);
  if (bwd)
    bn_reduce_kernel<T, true><<<sh.grid, sh.block, smem, s>>>(px, reinterpret_cast<const T*>(a.dy),
                                                              reinterpret_cast<const T*>(a.y_relu), a.save_mean, a.save_rstd, out,
                                                              a.M, a.C, rows_per_cta);
  else
    bn_reduce_kernel<T, false><<<sh.grid, sh.block, smem, s>>>(px, nullptr, nullptr, nullptr, nullptr, out, a.M, a.C, rows_per_cta);
  RT_LAUNCH_CHECK();
}

template <typename T>
void fwd_t(const BatchNormArgs& a, cudaStream_t s) {
  constexpr int V = VecN<T>::N;
  if (a.training) {
    RT_CUDA_CHECK(cudaMemsetAsync(a.scratch, 0, sizeof(float) * 2 * a.C, s));
    launch_reduce<T>(a, false, a.scratch, s);
  }
  const BnShape sh = bn_shape(a.M, a.C / V, 256, 4, 8);
  bn_apply_kernel<T><<<sh.grid, sh.block, 0, s>>>(
      reinterpret_cast<const T*>(a.x), reinterpret_cast<const T*>(a.residual), reinterpret_cast<T*>(a.y), a.scratch, a.gamma,
      a.beta, a.running_mean, a.running_var, a.save_mean, a.save_rstd, a.M, a.C, a.eps, a.momentum, a.relu, a.training);
  RT_LAUNCH_CHECK();
}

template <typename T>
void bwd_t(const BatchNormArgs& a, cudaStream_t s) {
  constexpr int V = VecN<T>::N;
  RT_CUDA_CHECK(cudaMemsetAsync(a.scratch, 0, sizeof(float) * 2 * a.C, s));
  launch_reduce<T>(a, true, a.scratch, s);
  const BnShape sh = bn_shape(a.M, a.C / V, 256, 2, 8);
  bn_bwd_apply_kernel<T><<<sh.grid, sh.block, 0, s>>>(
      reinterpret_cast<const T*>(a.x), reinterpret_cast<const T*>(a.dy), reinterpret_cast<const T*>(a.y_relu),
      reinterpret_cast<T*>(a.dx), reinterpret_cast<T*>(a.dres), a.scratch, a.save_mean, a.save_rstd, a.gamma, a.M, a.C);
  RT_LAUNCH_CHECK();
}

void check_args(const BatchNormArgs& a) {
  RT_CHECK(a.dtype >= DT_F32 && a.dtype <= DT_F16, "batchnorm: dtype must be fp32, bf16 or fp16");
  const int V = a.dtype == DT_F32 ? 4 : 8;
  RT_CHECK(a.C % V == 0, "batchnorm: channels must be a multiple of 8 (4 for fp32)");
  RT_CHECK(a.M > 0 && a.scratch != nullptr, "batchnorm: empty input or missing scratch");
}

}  // namespace

// scratch: fp32 [2][C].  Training: statistics of this batch; inference: running statistics.
void batchnorm_fwd(const BatchNormArgs& a, cudaStream_t s) {
  check_args(a);
  if (a.dtype == DT_F32) fwd_t<float>(a, s);
  else if (a.dtype == DT_BF16) fwd_t<__nv_bfloat16>(a, s);
  else fwd_t<__half>(a, s);
}

// After the call scratch holds [sum(dy), sum(dy * xhat)] = [dbeta, dgamma].
void batchnorm_bwd(const BatchNormArgs& a, cudaStream_t s) {
  check_args(a);
  RT_CHECK(a.save_mean && a.save_rstd && a.dy && a.dx, "batchnorm_bwd: saved statistics, dy and dx required");
  if (a.dtype == DT_F32) bwd_t<float>(a, s);
  else if (a.dtype == DT_BF16) bwd_t<__nv_bfloat16>(a, s);
  else bwd_t<__half>(a, s);
}

}  // namespace rt
