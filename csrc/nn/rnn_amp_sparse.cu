// Recurrent-cell gate kernels, the AMP unscale / overflow check, and CSR sparse x dense products.
//
//   lstm_gates   gates[B][4H] (order i, f, g, o; the sums x W_ih^T + h W_hh^T + b come from GEMMs) ->
//                c' = sigmoid(f) c + sigmoid(i) tanh(g),  h' = sigmoid(o) tanh(c'); the activated gates overwrite the
//                input so that the backward kernel needs nothing else.  Backward: (dh', dc') -> d(pre-activation
//                gates), dc.  Same math as the reference's cell (src/nn/lstm_cell.rs:84-126), one pass instead of a
//                dozen tensor ops.
//   gru_gates    gi[B][3H], gh[B][3H] (order r, z, n) -> r = s(gi_r + gh_r), z = s(gi_z + gh_z),
//                n = tanh(gi_n + r gh_n), h' = (1 - z) n + z h; backward gives d gi, d gh, dh (src/nn/gru_cell.rs).
//   amp_unscale  g *= inv_scale over a flat fp32 / bf16 / fp16 buffer and found_inf = 1 if any value is not finite
//                (src/amp/grad_scaler.rs unscale + check loops).
//   csr_spmm     y[rows][n] = A_csr x[cols][n], fp32: one warp per sparse row, lanes across dense columns
//                (n = 1 is SpMV with lanes across the row's non-zeros).  src/sparse/gpu_ops.rs:26-120.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

__device__ __forceinline__ float rf(float v) { return v; }
__device__ __forceinline__ float rf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float rf(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T rt_(float v);
template <> __device__ __forceinline__ float rt_<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 rt_<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half rt_<__half>(float v) { return __float2half(v); }
__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) lstm_fwd_kernel(T* __restrict__ gates, const T* __restrict__ c, T* __restrict__ h_out,
                                                       T* __restrict__ c_out, int B, int H) {
  const long long total = (long long)B * H;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(t / H), j = (int)(t % H);
    T* g = gates + (long long)b * 4 * H;
    const float i_ = sigm(rf(g[j])), f_ = sigm(rf(g[H + j])), g_ = tanhf(rf(g[2 * H + j])), o_ = sigm(rf(g[3 * H + j]));
    const float cn = f_ * rf(c[t]) + i_ * g_;
    g[j] = rt_<T>(i_); g[H + j] = rt_<T>(f_); g[2 * H + j] = rt_<T>(g_); g[3 * H + j] = rt_<T>(o_);
    c_out[t] = rt_<T>(cn);
    h_out[t] = rt_<T>(o_ * tanhf(cn));
  }
}

// act: activated gates from the forward pass; dgates receives the gradient of the pre-activation sums.
template <typename T>
__global__ void __launch_bounds__(256) lstm_bwd_kernel(const T* __restrict__ act, const T* __restrict__ c, const T* __restrict__ c_new,
                                                       const T* __restrict__ dh, const T* __restrict__ dc_new, T* __restrict__ dgates,
                                                       T* __restrict__ dc, int B, int H) {
  const long long total = (long long)B * H;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(t / H), j = (int)(t % H);
    const T* a = act + (long long)b * 4 * H;
    T* d = dgates + (long long)b * 4 * H;
    const float i_ = rf(a[j]), f_ = rf(a[H + j]), g_ = rf(a[2 * H + j]), o_ = rf(a[3 * H + j]);
    const float tc = tanhf(rf(c_new[t]));
    const float dhv = dh ? rf(dh[t]) : 0.f;
    const float dcn = (dc_new ? rf(dc_new[t]) : 0.f) + dhv * o_ * (1.f - tc * tc);
    d[j] = rt_<T>(dcn * g_ * i_ * (1.f - i_));
    d[H + j] = rt_<T>(dcn * rf(c[t]) * f_ * (1.f - f_));
    d[2 * H + j] = rt_<T>(dcn * i_ * (1.f - g_ * g_));
    d[3 * H + j] = rt_<T>(dhv * tc * o_ * (1.f - o_));
    dc[t] = rt_<T>(dcn * f_);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gru_fwd_kernel(const T* __restrict__ gi, const T* __restrict__ gh, const T* __restrict__ h,
                                                      T* __restrict__ h_out, T* __restrict__ save, int B, int H) {
  const long long total = (long long)B * H;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(t / H), j = (int)(t % H);
    const T* a = gi + (long long)b * 3 * H;
    const T* c = gh + (long long)b * 3 * H;
    const float r = sigm(rf(a[j]) + rf(c[j])), z = sigm(rf(a[H + j]) + rf(c[H + j]));
    const float hn = rf(c[2 * H + j]);
    const float n = tanhf(rf(a[2 * H + j]) + r * hn);
    h_out[t] = rt_<T>((1.f - z) * n + z * rf(h[t]));
    T* s = save + (long long)b * 4 * H;               // r, z, n, gh_n
    s[j] = rt_<T>(r); s[H + j] = rt_<T>(z); s[2 * H + j] = rt_<T>(n); s[3 * H + j] = rt_<T>(hn);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gru_bwd_kernel(const T* __restrict__ save, const T* __restrict__ h, const T* __restrict__ dh_new,
                                                      T* __restrict__ dgi, T* __restrict__ dgh, T* __restrict__ dh, int B, int H) {
  const long long total = (long long)B * H;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(t / H), j = (int)(t % H);
    const T* s = save + (long long)b * 4 * H;
    const float r = rf(s[j]), z = rf(s[H + j]), n = rf(s[2 * H + j]), hn = rf(s[3 * H + j]);
    const float g = rf(dh_new[t]);
    const float dn = g * (1.f - z) * (1.f - n * n);     // d(pre-activation of n)
    const float dz = g * (rf(h[t]) - n) * z * (1.f - z);
    const float dr = dn * hn * r * (1.f - r);
    T* a = dgi + (long long)b * 3 * H;
    T* c = dgh + (long long)b * 3 * H;
    a[j] = rt_<T>(dr); a[H + j] = rt_<T>(dz); a[2 * H + j] = rt_<T>(dn);
    c[j] = rt_<T>(dr); c[H + j] = rt_<T>(dz); c[2 * H + j] = rt_<T>(dn * r);
    dh[t] = rt_<T>(g * z);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) amp_unscale_kernel(T* __restrict__ g, long long n, float inv_scale, float* __restrict__ found_inf) {
  bool bad = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = rf(g[i]);
    if (!isfinite(v)) bad = true;
    g[i] = rt_<T>(v * inv_scale);
  }
  if (__syncthreads_or(bad ? 1 : 0) && threadIdx.x == 0) *found_inf = 1.f;
}

// One warp per sparse row.  n_dense == 1: lanes stride over the row's non-zeros and a shuffle sums them;
// otherwise lanes stride over dense columns and every lane walks the whole row.
__global__ void __launch_bounds__(256) csr_spmm_kernel(const long long* __restrict__ row_ptr, const long long* __restrict__ col,
                                                       const float* __restrict__ val, const float* __restrict__ x, float* __restrict__ y,
                                                       long long rows, int n_dense) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const long long b = row_ptr[r], e = row_ptr[r + 1];
    if (n_dense == 1) {
      float acc = 0.f;
      for (long long k = b + lane; k < e; k += 32) acc += val[k] * x[col[k]];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) y[r] = acc;
    } else {
      for (int j = lane; j < n_dense; j += 32) {
        float acc = 0.f;
        for (long long k = b; k < e; ++k) acc += val[k] * x[col[k] * n_dense + j];
        y[r * n_dense + j] = acc;
      }
    }
  }
}

int grid_of(long long work, int device) { return (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, 8LL * sm_count(device))); }

}  // namespace

#define RT_DISPATCH3(dtype, CALL)                         \
  do {                                                    \
    if ((dtype) == DT_F32) { using T = float; CALL; }     \
    else if ((dtype) == DT_BF16) { using T = __nv_bfloat16; CALL; } \
    else { using T = __half; CALL; }                      \
  } while (0)

void lstm_gates_fwd(int dtype, void* gates, const void* c, void* h_out, void* c_out, int B, int H, cudaStream_t s) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "lstm_gates: dtype must be fp32, bf16 or fp16");
  if ((long long)B * H == 0) return;
  const int grid = grid_of((long long)B * H, current_device());
  RT_DISPATCH3(dtype, (lstm_fwd_kernel<T><<<grid, 256, 0, s>>>((T*)gates, (const T*)c, (T*)h_out, (T*)c_out, B, H)));
  RT_LAUNCH_CHECK();
}

void lstm_gates_bwd(int dtype, const void* act, const void* c, const void* c_new, const void* dh, const void* dc_new, void* dgates,
                    void* dc, int B, int H, cudaStream_t s) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "lstm_gates: dtype must be fp32, bf16 or fp16");
  if ((long long)B * H == 0) return;
  const int grid = grid_of((long long)B * H, current_device());
  RT_DISPATCH3(dtype, (lstm_bwd_kernel<T><<<grid, 256, 0, s>>>((const T*)act, (const T*)c, (const T*)c_new, (const T*)dh,
                                                               (const T*)dc_new, (T*)dgates, (T*)dc, B, H)));
  RT_LAUNCH_CHECK();
}

void gru_gates_fwd(int dtype, const void* gi, const void* gh, const void* h, void* h_out, void* save, int B, int H, cudaStream_t s) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "gru_gates: dtype must be fp32, bf16 or fp16");
  if ((long long)B * H == 0) return;
  const int grid = grid_of((long long)B * H, current_device());
  RT_DISPATCH3(dtype, (gru_fwd_kernel<T><<<grid, 256, 0, s>>>((const T*)gi, (const T*)gh, (const T*)h, (T*)h_out, (T*)save, B, H)));
  RT_LAUNCH_CHECK();
}

void gru_gates_bwd(int dtype, const void* save, const void* h, const void* dh_new, void* dgi, void* dgh, void* dh, int B, int H,
                   cudaStream_t s) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "gru_gates: dtype must be fp32, bf16 or fp16");
  if ((long long)B * H == 0) return;
  const int grid = grid_of((long long)B * H, current_device());
  RT_DISPATCH3(dtype, (gru_bwd_kernel<T><<<grid, 256, 0, s>>>((const T*)save, (const T*)h, (const T*)dh_new, (T*)dgi, (T*)dgh, (T*)dh, B, H)));
  RT_LAUNCH_CHECK();
}

void amp_unscale(int dtype, void* grads, long long n, float inv_scale, float* found_inf, cudaStream_t s) {
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "amp_unscale: dtype must be fp32, bf16 or fp16");
  if (n == 0) return;
  const int grid = grid_of(n, current_device());
  RT_DISPATCH3(dtype, (amp_unscale_kernel<T><<<grid, 256, 0, s>>>((T*)grads, n, inv_scale, found_inf)));
  RT_LAUNCH_CHECK();
}

void csr_spmm(const long long* row_ptr, const long long* col, const float* val, const float* x, float* y, long long rows, int n_dense,
              cudaStream_t s) {
  RT_CHECK(n_dense >= 1, "csr_spmm: at least one dense column");
  if (rows == 0) return;
  const int grid = grid_of(rows * 32, current_device());
  csr_spmm_kernel<<<grid, 256, 0, s>>>(row_ptr, col, val, x, y, rows, n_dense);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
