// Elementwise arithmetic and activation kernels (forward and backward), fp32 / bf16 / fp16.
//
// Restates on the device the per-element math of the reference's CUDA-C string kernels and shader
// twins (src/gpu/cuda_kernels.rs:70-250 elementwise add/mul/relu/sigmoid/tanh/gelu; the Metal and OpenCL
// versions src/gpu/metal_shaders.metal:8-132, src/gpu/opencl_kernels.cl:5-289; activations
// src/nn/activation.rs:30-930).  The reference launches one thread per element with 4-byte accesses;
// here every thread moves 16 bytes per operand per step (8 x 16-bit or 4 x 32-bit values), the grid is
// sized to the SM count with a grid-stride loop, and math is done in fp32 whatever the storage type.
// These ops are HBM-bound: the roofline is (bytes read + bytes written) / copy bandwidth.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

template <typename T> struct Vec;  // 16-byte vector of T
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec<__half> { static constexpr int N = 8; };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[Vec<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) f[i] = to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[Vec<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) e[i] = from_f<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ------------------------------------------------------------------ op functors
__device__ __forceinline__ float binary_op(int op, float a, float b, float alpha) {
  switch (op) {
    case EW_ADD: return a + alpha * b;
    case EW_SUB: return a - alpha * b;
    case EW_MUL: return a * b;
    case EW_DIV: return a / b;
    case EW_MAX: return fmaxf(a, b);
    case EW_MIN: return fminf(a, b);
    case EW_POW: return powf(a, b);
    default: return 0.f;
  }
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_grad_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ float unary_op(int op, float x, float p0, float p1) {
  switch (op) {
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_SIGMOID: return sigmoid_f(x);
    case ACT_TANH: return tanhf(x);
    case ACT_GELU_TANH: return gelu_tanh_f(x);
    case ACT_GELU_ERF: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case ACT_SILU: return x * sigmoid_f(x);
    case ACT_ELU: return x > 0.f ? x : p0 * expm1f(x);
    case ACT_LEAKY_RELU: return x > 0.f ? x : p0 * x;
    case ACT_SELU: return 1.0507009873554805f * (x > 0.f ? x : 1.6732632423543772f * expm1f(x));
    case ACT_MISH: return x * tanhf(softplus_f(x));
    case ACT_SOFTPLUS: return p0 * x > p1 ? x : log1pf(__expf(p0 * x)) / p0;
    case ACT_HARDTANH: return fminf(fmaxf(x, p0), p1);
    case ACT_RELU6: return fminf(fmaxf(x, 0.f), 6.f);
    case ACT_HARDSIGMOID: return fminf(fmaxf(x * (1.f / 6.f) + 0.5f, 0.f), 1.f);
    case ACT_HARDSWISH: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) * (1.f / 6.f);
    case ACT_EXP: return __expf(x);
    case ACT_LOG: return __logf(x);
    case ACT_SQRT: return sqrtf(x);
    case ACT_RSQRT: return rsqrtf(x);
    case ACT_NEG: return -x;
    case ACT_ABS: return fabsf(x);
    case ACT_SQUARE: return x * x;
    case ACT_SIN: return sinf(x);
    case ACT_COS: return cosf(x);
    case ACT_SCALE_SHIFT: return x * p0 + p1;
    case ACT_RECIPROCAL: return 1.f / x;
    default: return x;
  }
}

// d(op)/dx evaluated from the forward INPUT x.
__device__ __forceinline__ float unary_grad(int op, float x, float p0, float p1) {
  switch (op) {
    case ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case ACT_SIGMOID: { const float s = sigmoid_f(x); return s * (1.f - s); }
    case ACT_TANH: { const float t = tanhf(x); return 1.f - t * t; }
    case ACT_GELU_TANH: return gelu_tanh_grad_f(x);
    case ACT_GELU_ERF: return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    case ACT_SILU: { const float s = sigmoid_f(x); return s * (1.f + x * (1.f - s)); }
    case ACT_ELU: return x > 0.f ? 1.f : p0 * __expf(x);
    case ACT_LEAKY_RELU: return x > 0.f ? 1.f : p0;
    case ACT_SELU: return 1.0507009873554805f * (x > 0.f ? 1.f : 1.6732632423543772f * __expf(x));
    case ACT_MISH: {
      const float sp = softplus_f(x), t = tanhf(sp);
      return t + x * (1.f - t * t) * sigmoid_f(x);
    }
    case ACT_SOFTPLUS: return p0 * x > p1 ? 1.f : sigmoid_f(p0 * x);
    case ACT_HARDTANH: return (x > p0 && x < p1) ? 1.f : 0.f;
    case ACT_RELU6: return (x > 0.f && x < 6.f) ? 1.f : 0.f;
    case ACT_HARDSIGMOID: return (x > -3.f && x < 3.f) ? (1.f / 6.f) : 0.f;
    case ACT_HARDSWISH: return x <= -3.f ? 0.f : (x >= 3.f ? 1.f : (2.f * x + 3.f) * (1.f / 6.f));
    case ACT_EXP: return __expf(x);
    case ACT_LOG: return 1.f / x;
    case ACT_SQRT: return 0.5f * rsqrtf(x);
    case ACT_RSQRT: return -0.5f * rsqrtf(x) / x;
    case ACT_NEG: return -1.f;
    case ACT_ABS: return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f);
    case ACT_SQUARE: return 2.f * x;
    case ACT_SIN: return cosf(x);
    case ACT_COS: return -sinf(x);
    case ACT_SCALE_SHIFT: return p0;
    case ACT_RECIPROCAL: return -1.f / (x * x);
    default: return 1.f;
  }
}

// ------------------------------------------------------------------ kernels
// mode 0: out = op(a, b); 1: out = op(a, scalar); 2: out = op(scalar, a)
template <typename T, int OP>
__global__ void __launch_bounds__(256) binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                     long long n, float scalar, float alpha, int mode) {
  constexpr int V = Vec<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float fa[V], fb[V], fo[V];
    load_vec(a + i * V, fa);
    if (mode == 0) load_vec(b + i * V, fb);
#pragma unroll
    for (int e = 0; e < V; ++e)
      fo[e] = mode == 0 ? binary_op(OP, fa[e], fb[e], alpha)
                        : (mode == 1 ? binary_op(OP, fa[e], scalar, alpha) : binary_op(OP, scalar, fa[e], alpha));
    store_vec(out + i * V, fo);
  }
  // tail (n not a multiple of the vector width)
  const long long t = nvec * V + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) {
    const float x = to_f(a[t]);
    const float y = mode == 0 ? to_f(b[t]) : scalar;
    out[t] = from_f<T>(mode == 2 ? binary_op(OP, y, x, alpha) : binary_op(OP, x, y, alpha));
  }
}

template <typename T, int OP, bool BWD>
__global__ void __launch_bounds__(256) unary_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out,
                                                    long long n, float p0, float p1) {
  constexpr int V = Vec<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float fx[V], fg[V], fo[V];
    load_vec(x + i * V, fx);
    if (BWD) load_vec(dy + i * V, fg);
#pragma unroll
    for (int e = 0; e < V; ++e) fo[e] = BWD ? fg[e] * unary_grad(OP, fx[e], p0, p1) : unary_op(OP, fx[e], p0, p1);
    store_vec(out + i * V, fo);
  }
  const long long t = nvec * V + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) {
    const float v = to_f(x[t]);
    out[t] = from_f<T>(BWD ? to_f(dy[t]) * unary_grad(OP, v, p0, p1) : unary_op(OP, v, p0, p1));
  }
}

inline unsigned ew_grid(long long nvec, int device) {
  const long long want = (nvec + 255) / 256;
  const long long cap = (long long)sm_count(device) * 8;
  return (unsigned)std::max<long long>(1, std::min(want, cap));
}

template <typename T, int OP>
void launch_binary_t(const void* a, const void* b, void* out, long long n, float scalar, float alpha, int mode,
                     int device, cudaStream_t s) {
  binary_kernel<T, OP><<<ew_grid(n / Vec<T>::N + 1, device), 256, 0, s>>>(
      reinterpret_cast<const T*>(a), reinterpret_cast<const T*>(b), reinterpret_cast<T*>(out), n, scalar, alpha, mode);
}

template <int OP>
void launch_binary_op(int dtype, const void* a, const void* b, void* out, long long n, float scalar, float alpha,
                      int mode, int device, cudaStream_t s) {
  if (dtype == DT_F32) launch_binary_t<float, OP>(a, b, out, n, scalar, alpha, mode, device, s);
  else if (dtype == DT_BF16) launch_binary_t<__nv_bfloat16, OP>(a, b, out, n, scalar, alpha, mode, device, s);
  else launch_binary_t<__half, OP>(a, b, out, n, scalar, alpha, mode, device, s);
}

template <typename T, int OP>
void launch_unary_t(const void* x, const void* dy, void* out, long long n, float p0, float p1, bool bwd, int device,
                    cudaStream_t s) {
  const unsigned grid = ew_grid(n / Vec<T>::N + 1, device);
  if (bwd)
    unary_kernel<T, OP, true><<<grid, 256, 0, s>>>(reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(dy),
                                                   reinterpret_cast<T*>(out), n, p0, p1);
  else
    unary_kernel<T, OP, false><<<grid, 256, 0, s>>>(reinterpret_cast<const T*>(x), nullptr, reinterpret_cast<T*>(out),
                                                    n, p0, p1);
}

template <int OP>
void launch_unary_op(int dtype, const void* x, const void* dy, void* out, long long n, float p0, float p1, bool bwd,
                     int device, cudaStream_t s) {
  if (dtype == DT_F32) launch_unary_t<float, OP>(x, dy, out, n, p0, p1, bwd, device, s);
  else if (dtype == DT_BF16) launch_unary_t<__nv_bfloat16, OP>(x, dy, out, n, p0, p1, bwd, device, s);
  else launch_unary_t<__half, OP>(x, dy, out, n, p0, p1, bwd, device, s);
}

void check_ptrs(const void* a, const void* b, const void* c) {
  RT_CHECK(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0,
           "elementwise: operands must be 16-byte aligned");
}

}  // namespace

void elementwise_binary(int op, int dtype, const void* a, const void* b, void* out, long long n, float scalar,
                        float alpha, int mode, cudaStream_t s) {
  if (n == 0) return;
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "elementwise_binary: dtype must be fp32, bf16 or fp16");
  RT_CHECK(mode >= 0 && mode <= 2, "elementwise_binary: bad mode");
  check_ptrs(a, mode == 0 ? b : nullptr, out);
  const int dev = current_device();
#define RT_BIN(OP) case OP: launch_binary_op<OP>(dtype, a, b, out, n, scalar, alpha, mode, dev, s); break;
  switch (op) {
    RT_BIN(EW_ADD) RT_BIN(EW_SUB) RT_BIN(EW_MUL) RT_BIN(EW_DIV) RT_BIN(EW_MAX) RT_BIN(EW_MIN) RT_BIN(EW_POW)
    default: fail("elementwise_binary: unknown op");
  }
#undef RT_BIN
  RT_LAUNCH_CHECK();
}

void elementwise_unary(int op, int dtype, const void* x, const void* dy, void* out, long long n, float p0, float p1,
                       bool backward, cudaStream_t s) {
  if (n == 0) return;
  RT_CHECK(dtype >= DT_F32 && dtype <= DT_F16, "elementwise_unary: dtype must be fp32, bf16 or fp16");
  RT_CHECK(!backward || dy != nullptr, "elementwise_unary: backward needs dy");
  check_ptrs(x, dy, out);
  const int dev = current_device();
#define RT_UN(OP) case OP: launch_unary_op<OP>(dtype, x, dy, out, n, p0, p1, backward, dev, s); break;
  switch (op) {
    RT_UN(ACT_RELU) RT_UN(ACT_SIGMOID) RT_UN(ACT_TANH) RT_UN(ACT_GELU_TANH) RT_UN(ACT_GELU_ERF) RT_UN(ACT_SILU)
    RT_UN(ACT_ELU) RT_UN(ACT_LEAKY_RELU) RT_UN(ACT_SELU) RT_UN(ACT_MISH) RT_UN(ACT_SOFTPLUS) RT_UN(ACT_HARDTANH)
    RT_UN(ACT_RELU6) RT_UN(ACT_HARDSIGMOID) RT_UN(ACT_HARDSWISH) RT_UN(ACT_EXP) RT_UN(ACT_LOG) RT_UN(ACT_SQRT)
    RT_UN(ACT_RSQRT) RT_UN(ACT_NEG) RT_UN(ACT_ABS) RT_UN(ACT_SQUARE) RT_UN(ACT_SIN) RT_UN(ACT_COS)
    RT_UN(ACT_SCALE_SHIFT) RT_UN(ACT_RECIPROCAL)
    default: fail("elementwise_unary: unknown op");
  }
#undef RT_UN
  RT_LAUNCH_CHECK();
}

}  // namespace rt
