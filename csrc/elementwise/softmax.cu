// Row softmax / log-softmax (forward, backward) and row reductions over the last dimension.
//
// The reference computes softmax with scalar host loops (src/nn/activation.rs:423-520) and reductions with
// a two-stage shared-memory tree per block (K8, src/gpu/cuda_kernels.rs:252-330).  Here one warp owns a row
// while the row fits its registers (C <= 1024: a single pass over HBM, 16-byte loads, shuffle reductions),
// and one CTA owns a row beyond that (online max/sum in the first pass, second pass writes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

__device__ __forceinline__ float ldf(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float ldf(const __half* p, long long i) { return __half2float(p[i]); }
__device__ __forceinline__ void stf(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }
__device__ __forceinline__ void stf(__half* p, long long i, float v) { p[i] = __float2half(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

// CTA-wide reduction helpers (blockDim.x multiple of 32, <= 1024); `red` has 32 floats.
template <int MODE>  // 0 sum, 1 max, 2 min
__device__ __forceinline__ float block_reduce(float v, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  v = MODE == 0 ? warp_sum(v) : (MODE == 1 ? warp_max(v) : warp_min(v));
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : (MODE == 0 ? 0.f : (MODE == 1 ? -CUDART_INF_F : CUDART_INF_F));
  r = MODE == 0 ? warp_sum(r) : (MODE == 1 ? warp_max(r) : warp_min(r));
  return r;
}

// One warp per row, the row cached in registers: PER lane elements, C <= 32 * PER.
template <typename T, int PER, bool BWD>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                           long long rows, int C, long long ld, int log_mode) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* pa = a + row * ld;
  const T* pb = BWD ? b + row * ld : nullptr;
  T* po = out + row * ld;
  float va[PER], vb[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = lane + 32 * i;
    va[i] = c < C ? ldf(pa, c) : (BWD ? 0.f : -CUDART_INF_F);
    if (BWD) vb[i] = c < C ? ldf(pb, c) : 0.f;
  }
  if (!BWD) {
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < PER; ++i) mx = fmaxf(mx, va[i]);
    mx = warp_max(mx);
    if (mx == -CUDART_INF_F) mx = 0.f;  // fully masked row
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      va[i] = log_mode ? va[i] - mx : __expf(va[i] - mx);
      sum += log_mode ? __expf(va[i]) : va[i];
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f, lg = __logf(sum);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = lane + 32 * i;
      if (c < C) stf(po, c, log_mode ? va[i] - lg : va[i] * inv);
    }
  } else {
    // a = y (forward output), b = dy
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) dot += log_mode ? vb[i] : vb[i] * va[i];
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = lane + 32 * i;
      if (c < C) stf(po, c, log_mode ? vb[i] - __expf(va[i]) * dot : va[i] * (vb[i] - dot));
    }
  }
}

// One CTA per row for long rows.
template <typename T, bool BWD>
__global__ void __launch_bounds__(512) softmax_block_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                            int C, long long ld, int log_mode) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* pa = a + row * ld;
  const T* pb = BWD ? b + row * ld : nullptr;
  T* po = out + row * ld;
  if (!BWD) {
    float mx = -CUDART_INF_F, sum = 0.f;  // online max / sum
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float v = ldf(pa, c);
      if (v > mx) {
        sum = sum * __expf(mx - v) + 1.f;
        mx = v;
      } else if (v != -CUDART_INF_F) {
        sum += __expf(v - mx);
      }
    }
    const float gmx = block_reduce<1>(mx, red);
    const float m0 = gmx == -CUDART_INF_F ? 0.f : gmx;
    sum = mx == -CUDART_INF_F ? 0.f : sum * __expf(mx - m0);
    const float gsum = block_reduce<0>(sum, red);
    const float inv = gsum > 0.f ? 1.f / gsum : 0.f, lg = __logf(gsum);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float v = ldf(pa, c) - m0;
      stf(po, c, log_mode ? v - lg : __expf(v) * inv);
    }
  } else {
    float dot = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) dot += log_mode ? ldf(pb, c) : ldf(pb, c) * ldf(pa, c);
    dot = block_reduce<0>(dot, red);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float y = ldf(pa, c), g = ldf(pb, c);
      stf(po, c, log_mode ? g - __expf(y) * dot : y * (g - dot));
    }
  }
}

template <typename T, bool BWD>
void launch_softmax(const void* a, const void* b, void* out, long long rows, int C, long long ld, int log_mode, cudaStream_t s) {
  auto pa = reinterpret_cast<const T*>(a);
  auto pb = reinterpret_cast<const T*>(b);
  auto po = reinterpret_cast<T*>(out);
  const unsigned wgrid = (unsigned)((rows + 7) / 8);
  if (C <= 128) softmax_warp_kernel<T, 4, BWD><<<wgrid, 256, 0, s>>>(pa, pb, po, rows, C, ld, log_mode);
  else if (C <= 256) softmax_warp_kernel<T, 8, BWD><<<wgrid, 256, 0, s>>>(pa, pb, po, rows, C, ld, log_mode);
  else if (C <= 512) softmax_warp_kernel<T, 16, BWD><<<wgrid, 256, 0, s>>>(pa, pb, po, rows, C, ld, log_mode);
  else if (C <= 1024) softmax_warp_kernel<T, 32, BWD><<<wgrid, 256, 0, s>>>(pa, pb, po, rows, C, ld, log_mode);
  else softmax_block_kernel<T, BWD><<<(unsigned)rows, 512, 0, s>>>(pa, pb, po, C, ld, log_mode);
}

// mode: 0 sum, 1 mean, 2 max, 3 min, 4 variance
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int C,
                                                          long long ld, int mode, float unbiased) {
  // one warp per row
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* p = x + row * ld;
  float r;
  if (mode == 2 || mode == 3) {
    r = mode == 2 ? -CUDART_INF_F : CUDART_INF_F;
    for (int c = lane; c < C; c += 32) r = mode == 2 ? fmaxf(r, ldf(p, c)) : fminf(r, ldf(p, c));
    r = mode == 2 ? warp_max(r) : warp_min(r);
  } else if (mode == 4) {
    // Welford per lane, merged across lanes (Chan et al.)
    float n = 0.f, mean = 0.f, m2 = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float v = ldf(p, c);
      n += 1.f;
      const float d = v - mean;
      mean += d / n;
      m2 += d * (v - mean);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      const float n2 = __shfl_xor_sync(0xffffffffu, n, s), mean2 = __shfl_xor_sync(0xffffffffu, mean, s),
                  m22 = __shfl_xor_sync(0xffffffffu, m2, s);
      const float nt = n + n2;
      if (nt > 0.f) {
        const float d = mean2 - mean;
        mean += d * n2 / nt;
        m2 += m22 + d * d * n * n2 / nt;
      }
      n = nt;
    }
    const float den = unbiased != 0.f ? n - 1.f : n;
    r = den > 0.f ? m2 / den : CUDART_NAN_F;
  } else {
    r = 0.f;
    for (int c = lane; c < C; c += 32) r += ldf(p, c);
    r = warp_sum(r);
    if (mode == 1) r /= (float)C;
  }
  if (lane == 0) out[row] = r;
}

}  // namespace

void softmax_rows_fwd(int dtype, const void* x, void* y, long long rows, int C, long long ld, int log_mode, cudaStream_t s) {
  if (rows == 0 || C == 0) return;
  if (dtype == DT_F32) launch_softmax<float, false>(x, nullptr, y, rows, C, ld, log_mode, s);
  else if (dtype == DT_BF16) launch_softmax<__nv_bfloat16, false>(x, nullptr, y, rows, C, ld, log_mode, s);
  else if (dtype == DT_F16) launch_softmax<__half, false>(x, nullptr, y, rows, C, ld, log_mode, s);
  else fail("softmax_rows_fwd: dtype must be fp32, bf16 or fp16");
  RT_LAUNCH_CHECK();
}

void softmax_rows_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int C, long long ld, int log_mode,
                      cudaStream_t s) {
  if (rows == 0 || C == 0) return;
  if (dtype == DT_F32) launch_softmax<float, true>(y, dy, dx, rows, C, ld, log_mode, s);
  else if (dtype == DT_BF16) launch_softmax<__nv_bfloat16, true>(y, dy, dx, rows, C, ld, log_mode, s);
  else if (dtype == DT_F16) launch_softmax<__half, true>(y, dy, dx, rows, C, ld, log_mode, s);
  else fail("softmax_rows_bwd: dtype must be fp32, bf16 or fp16");
  RT_LAUNCH_CHECK();
}

void reduce_rows(int dtype, const void* x, float* out, long long rows, int C, long long ld, int mode, float p0, cudaStream_t s) {
  if (rows == 0) return;
  RT_CHECK(mode >= 0 && mode <= 4, "reduce_rows: bad mode");
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == DT_F32) reduce_rows_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<const float*>(x), out, rows, C, ld, mode, p0);
  else if (dtype == DT_BF16)
    reduce_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, rows, C, ld, mode, p0);
  else if (dtype == DT_F16)
    reduce_rows_kernel<__half><<<grid, 256, 0, s>>>(reinterpret_cast<const __half*>(x), out, rows, C, ld, mode, p0);
  else fail("reduce_rows: dtype must be fp32, bf16 or fp16");
  RT_LAUNCH_CHECK();
}

}  // namespace rt
