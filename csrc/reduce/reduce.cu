// Reductions used by training: column sums (bias gradients), sum of squares (gradient norm),
// plus the generic full reduce that restates the reference's reduce_sum_f32
// (src/gpu/cuda_kernels.cu:106-130) with warp shuffles and a single atomic per CTA.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

// out[n] += sum_m x[m][n]   x bf16 [M][ld], out fp32.  Thread owns 2 adjacent columns.
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                              long long M, int N, long long ld, int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= N) return;
  const long long m0 = (long long)blockIdx.y * rows_per_block;
  const long long m1 = min(M, m0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (c + 1 < N) {
    for (long long m = m0; m < m1; ++m) {
      float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + m * ld + c));
      a0 += v.x;
      a1 += v.y;
    }
    atomicAdd(out + c, a0);
    atomicAdd(out + c + 1, a1);
  } else {
    for (long long m = m0; m < m1; ++m) a0 += __bfloat162float(x[m * ld + c]);
    atomicAdd(out + c, a0);
  }
}

void colsum_accum(const void* x, float* out, long long M, int N, long long ld,
                  cudaStream_t stream) {
  RT_CHECK(ld % 2 == 0, "colsum: row stride must be even");
  if (M == 0 || N == 0) return;
  const int threads = 128;
  const int gx = ((N + 1) / 2 + threads - 1) / threads;
  int rpb = 256;
  long long gy = (M + rpb - 1) / rpb;
  dim3 grid(gx, (unsigned)gy);
  colsum_kernel<<<grid, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, M, N,
                                              ld, rpb);
  RT_LAUNCH_CHECK();
}

template <typename T, int MODE>  // MODE 0: sum, 1: sum of squares, 2: max, 3: min
__global__ void reduce_kernel(const T* __restrict__ x, float* __restrict__ out, long long n) {
  float acc = (MODE == 2) ? -INFINITY : (MODE == 3 ? INFINITY : 0.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = static_cast<float>(x[i]);
    if (MODE == 0) acc += v;
    else if (MODE == 1) acc += v * v;
    else if (MODE == 2) acc = fmaxf(acc, v);
    else acc = fminf(acc, v);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, acc, s);
    if (MODE <= 1) acc += o;
    else if (MODE == 2) acc = fmaxf(acc, o);
    else acc = fminf(acc, o);
  }
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    float t = lane < nw ? red[lane] : ((MODE == 2) ? -INFINITY : (MODE == 3 ? INFINITY : 0.f));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      const float o = __shfl_xor_sync(0xffffffffu, t, s);
      if (MODE <= 1) t += o;
      else if (MODE == 2) t = fmaxf(t, o);
      else t = fminf(t, o);
    }
    if (lane == 0) {
      if (MODE <= 1) atomicAdd(out, t);
      else if (MODE == 2) {
        // float max via int ordering trick on the sign
        int* oi = reinterpret_cast<int*>(out);
        if (t >= 0.f) atomicMax(oi, __float_as_int(t));
        else atomicMin(reinterpret_cast<unsigned int*>(oi), __float_as_uint(t));
      } else {
        int* oi = reinterpret_cast<int*>(out);
        if (t >= 0.f) atomicMin(oi, __float_as_int(t));
        else atomicMax(reinterpret_cast<unsigned int*>(oi), __float_as_uint(t));
      }
    }
  }
}

// out must be pre-initialised by the caller (0 for sums, -inf / +inf for max / min).
void reduce_all(const void* x, int dtype, int mode, float* out, long long n, cudaStream_t stream) {
  if (n == 0) return;
  const int threads = 256;
  const int grid = (int)std::min<long long>((n + threads - 1) / threads, 4LL * sm_count(current_device()));
#define RT_RED(T, M) reduce_kernel<T, M><<<grid, threads, 0, stream>>>(reinterpret_cast<const T*>(x), out, n)
  if (dtype == 0) {  // fp32
    if (mode == 0) RT_RED(float, 0); else if (mode == 1) RT_RED(float, 1);
    else if (mode == 2) RT_RED(float, 2); else RT_RED(float, 3);
  } else {  // bf16
    if (mode == 0) RT_RED(__nv_bfloat16, 0); else if (mode == 1) RT_RED(__nv_bfloat16, 1);
    else if (mode == 2) RT_RED(__nv_bfloat16, 2); else RT_RED(__nv_bfloat16, 3);
  }
#undef RT_RED
  RT_LAUNCH_CHECK();
}

}  // namespace rt
