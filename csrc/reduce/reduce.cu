// Reductions used by training: column sums (bias gradients), sum of squares (gradient norm),
// plus the generic full reduce that restates the reference's reduce_sum_f32
// (src/gpu/cuda_kernels.cu:106-130) with warp shuffles and a single atomic per CTA.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

// out[n] += sum_m x[m][n]   x bf16 [M][ld], out fp32.
// Block = 32 column groups (8 columns = one 16-byte load each) x 8 row lanes; a warp reads 512
// contiguous bytes of one row.  Row lanes are combined through shared memory, then one fp32
// atomic per column per block.
__global__ void colsum_vec_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                  long long M, int N, long long ld, int rows_per_block) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  __shared__ float part[8][32 * 8 + 8];
  const int cg = threadIdx.x & 31;
  const int rl = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + cg) * 8;
  const long long m0 = (long long)blockIdx.y * rows_per_block;
  const long long m1 = min(M, m0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (c0 < N) {
#pragma unroll 4
    for (long long m = m0 + rl; m < m1; m += 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(x + m * ld + c0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) part[rl][cg * 8 + e] = acc[e];
  __syncthreads();
  const int c = threadIdx.x;  // 256 threads -> 256 columns of this block
  const int col = blockIdx.x * 256 + c;
  if (col < N) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += part[r][c];
    atomicAdd(out + col, t);
  }
}

// Scalar fallback for N % 8 != 0 or unaligned rows: thread owns one column.
__global__ void colsum_scalar_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                     long long M, int N, long long ld, int rows_per_block) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  const long long m0 = (long long)blockIdx.y * rows_per_block;
  const long long m1 = min(M, m0 + rows_per_block);
  float a0 = 0.f;
  for (long long m = m0; m < m1; ++m) a0 += __bfloat162float(x[m * ld + c]);
  atomicAdd(out + c, a0);
}

void colsum_accum(const void* x, float* out, long long M, int N, long long ld,
                  cudaStream_t stream) {
  if (M == 0 || N == 0) return;
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  const bool vec = (N % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec) {
    const int gx = (N + 255) / 256;
    // enough blocks to cover the machine a few times over
    int rpb = 512;
    while (rpb > 64 && (long long)gx * ((M + rpb - 1) / rpb) < 4LL * sm_count(current_device())) rpb >>= 1;
    dim3 grid(gx, (unsigned)((M + rpb - 1) / rpb));
    colsum_vec_kernel<<<grid, 256, 0, stream>>>(xp, out, M, N, ld, rpb);
  } else {
    const int rpb = 256;
    dim3 grid((N + 127) / 128, (unsigned)((M + rpb - 1) / rpb));
    colsum_scalar_kernel<<<grid, 128, 0, stream>>>(xp, out, M, N, ld, rpb);
  }
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
