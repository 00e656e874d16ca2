// Multi-tensor optimizer step: ONE launch updates up to 32 parameter tensors (any sizes) with the rule of
// NAdam, RAdam, Adamax, RMSprop, AdaGrad, AdaBound or LAMB (plus Adam / AdamW / SGD for lists that do not live in a
// flat buffer).  The tensor table travels in the kernel parameters, so nothing is copied to the device per step;
// lists longer than 32 tensors take several launches.  Work is cut into chunks of 4096 elements; a CTA finds its
// (tensor, chunk) by a search over at most 33 prefix counts.  Parameters and gradients may be fp32 or bf16, the
// optimizer state is fp32.
//
// The per-step scalars that depend on the step count (bias corrections, NAdam's momentum schedule, RAdam's
// rectification term, AdaBound's clip interval) are computed on the host once per step and passed as c0..c3:
// the reference evaluates them per tensor inside its host loops (src/optim/nadam.rs:13-182,
// src/optim/radam.rs:13-239, src/optim/adamax.rs:13-178, src/optim/adabound.rs:19-78, src/optim/lamb.rs:19-82,
// src/optim/mod.rs:408-755).  LAMB takes two launches: phase 1 updates the moments and accumulates |w|^2 and
// |update|^2 per tensor into a small fp32 table, phase 2 applies the trust ratio.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

constexpr int MT_CHUNK = 4096;
constexpr int MT_THREADS = 256;

template <typename T>
__device__ __forceinline__ float mt_load(const T* p, long long i);
template <>
__device__ __forceinline__ float mt_load<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float mt_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void mt_store(T* p, long long i, float v);
template <>
__device__ __forceinline__ void mt_store<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void mt_store<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// Updates one element.  Returns the LAMB update direction (unused elsewhere).
__device__ __forceinline__ float mt_update(const MultiTensorArgs& a, float& p, float g, float& s0, float& s1, float& s2) {
  g *= a.grad_scale;
  if (a.maximize) g = -g;
  switch (a.mode) {
    case MT_ADAM:
    case MT_ADAMW: {
      if (a.mode == MT_ADAM) g += a.weight_decay * p;
      else p *= (1.f - a.lr * a.weight_decay);
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      p -= a.lr * (s0 / a.c0) / (sqrtf(s1 / a.c1) + a.eps);  // c0 = 1 - beta1^t, c1 = 1 - beta2^t
      return 0.f;
    }
    case MT_SGD: {  // beta1 = momentum, beta2 = dampening, c0 != 0 on the first step (buffer = gradient), c1 = nesterov
      g += a.weight_decay * p;
      float d = g;
      if (a.beta1 != 0.f) {
        s0 = (a.c0 != 0.f) ? g : (a.beta1 * s0 + (1.f - a.beta2) * g);
        d = (a.c1 != 0.f) ? (g + a.beta1 * s0) : s0;
      }
      p -= a.lr * d;
      return 0.f;
    }
    case MT_NADAM: {  // c0 = lr (1 - mu_t) / (1 - prod mu), c1 = lr mu_{t+1} / (1 - prod mu * mu_{t+1}), c2 = 1 - beta2^t
      if (a.decoupled) p *= (1.f - a.lr * a.weight_decay);
      else g += a.weight_decay * p;
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      const float denom = sqrtf(s1 / a.c2) + a.eps;
      p -= a.c0 * g / denom;
      p -= a.c1 * s0 / denom;
      return 0.f;
    }
    case MT_RADAM: {  // c0 = 1 - beta1^t, c1 = rectification (0: variance not tractable yet), c2 = sqrt(1 - beta2^t)
      if (a.decoupled) p *= (1.f - a.lr * a.weight_decay);
      else g += a.weight_decay * p;
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      const float mhat = s0 / a.c0;
      if (a.c1 > 0.f) p -= a.lr * mhat * a.c1 * a.c2 / (sqrtf(s1) + a.eps);
      else p -= a.lr * mhat;
      return 0.f;
    }
    case MT_ADAMAX: {  // s1 = exponentially weighted infinity norm, c0 = 1 - beta1^t
      g += a.weight_decay * p;
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = fmaxf(a.beta2 * s1, fabsf(g) + a.eps);
      p -= (a.lr / a.c0) * s0 / s1;
      return 0.f;
    }
    case MT_RMSPROP: {  // beta2 = alpha, beta1 = momentum, c0 != 0: centered; s0 = momentum buffer, s1 = square avg, s2 = grad avg
      g += a.weight_decay * p;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      float avg;
      if (a.c0 != 0.f) {
        s2 = a.beta2 * s2 + (1.f - a.beta2) * g;
        avg = sqrtf(fmaxf(s1 - s2 * s2, 0.f)) + a.eps;
      } else {
        avg = sqrtf(s1) + a.eps;
      }
      if (a.beta1 > 0.f) {
        s0 = a.beta1 * s0 + g / avg;
        p -= a.lr * s0;
      } else {
        p -= a.lr * g / avg;
      }
      return 0.f;
    }
    case MT_ADAGRAD: {  // c0 = lr / (1 + (t - 1) lr_decay); s1 = sum of squares
      g += a.weight_decay * p;
      s1 += g * g;
      p -= a.c0 * g / (sqrtf(s1) + a.eps);
      return 0.f;
    }
    case MT_ADABOUND: {  // c0 = lr sqrt(1 - beta2^t) / (1 - beta1^t), c1 / c2 = lower / upper bound of the step size
      g += a.weight_decay * p;
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      const float eta = fminf(fmaxf(a.c0 / (sqrtf(s1) + a.eps), a.c1), a.c2);
      p -= eta * s0;
      return 0.f;
    }
    case MT_LAMB_STAGE1: {  // c0 = 1 - beta1^t (or 1), c1 = 1 - beta2^t (or 1); p untouched
      s0 = a.beta1 * s0 + (1.f - a.beta1) * g;
      s1 = a.beta2 * s1 + (1.f - a.beta2) * g * g;
      return (s0 / a.c0) / (sqrtf(s1 / a.c1) + a.eps) + a.weight_decay * p;
    }
    default:
      return 0.f;
  }
}

template <typename TP, typename TG>
__global__ void __launch_bounds__(MT_THREADS) multi_tensor_optim_kernel(const MultiTensorArgs a) {
  // which tensor does this chunk belong to?
  int t = 0;
#pragma unroll 1
  while (t + 1 < a.n_tensors && int(blockIdx.x) >= a.chunk_start[t + 1]) ++t;
  const long long begin = (long long)(int(blockIdx.x) - a.chunk_start[t]) * MT_CHUNK;
  const long long end = min(a.numel[t], begin + MT_CHUNK);
  TP* P = reinterpret_cast<TP*>(a.param[t]);
  const TG* G = reinterpret_cast<const TG*>(a.grad[t]);
  float* S0 = a.state0[t];
  float* S1 = a.state1[t];
  float* S2 = a.state2[t];
  float w2 = 0.f, u2 = 0.f;
  float trust = 1.f;
  if (a.mode == MT_LAMB_STAGE2) {
    const float wn = sqrtf(a.norms[2 * (a.tensor_base + t)]), un = sqrtf(a.norms[2 * (a.tensor_base + t) + 1]);
    trust = (wn > 0.f && un > 0.f) ? wn / un : 1.f;
  }
  for (long long i = begin + threadIdx.x; i < end; i += MT_THREADS) {
    float p = mt_load<TP>(P, i);
    float s0 = S0 ? S0[i] : 0.f, s1 = S1 ? S1[i] : 0.f, s2 = S2 ? S2[i] : 0.f;
    if (a.mode == MT_LAMB_STAGE2) {  // moments are already updated: rebuild the direction and apply it
      const float upd = (s0 / a.c0) / (sqrtf(s1 / a.c1) + a.eps) + a.weight_decay * p;
      p -= a.lr * trust * upd;
      mt_store<TP>(P, i, p);
      continue;
    }
    const float g = mt_load<TG>(G, i);
    const float upd = mt_update(a, p, g, s0, s1, s2);
    if (S0) S0[i] = s0;
    if (S1) S1[i] = s1;
    if (S2) S2[i] = s2;
    if (a.mode == MT_LAMB_STAGE1) {
      w2 += p * p;
      u2 += upd * upd;
    } else {
      mt_store<TP>(P, i, p);
    }
  }
  if (a.mode == MT_LAMB_STAGE1) {
    __shared__ float red[2][MT_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      w2 += __shfl_xor_sync(0xffffffffu, w2, o);
      u2 += __shfl_xor_sync(0xffffffffu, u2, o);
    }
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = w2;
      red[1][threadIdx.x >> 5] = u2;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int k = 0; k < MT_THREADS / 32; ++k) {
        a0 += red[0][k];
        a1 += red[1][k];
      }
      atomicAdd(&a.norms[2 * (a.tensor_base + t)], a0);
      atomicAdd(&a.norms[2 * (a.tensor_base + t) + 1], a1);
    }
  }
}

void multi_tensor_optim_step(MultiTensorArgs& a, cudaStream_t stream) {
  RT_CHECK(a.n_tensors >= 0 && a.n_tensors <= MT_MAX_TENSORS, "multi_tensor_optim: at most 32 tensors per launch");
  if (a.n_tensors == 0) return;
  RT_CHECK(a.mode >= MT_ADAM && a.mode <= MT_LAMB_STAGE2, "multi_tensor_optim: unknown update rule");
  RT_CHECK((a.mode != MT_LAMB_STAGE1 && a.mode != MT_LAMB_STAGE2) || a.norms != nullptr, "multi_tensor_optim: LAMB needs the norm table");
  int chunks = 0;
  for (int t = 0; t < a.n_tensors; ++t) {
    RT_CHECK(a.numel[t] >= 0 && a.param[t] != nullptr, "multi_tensor_optim: bad tensor entry");
    a.chunk_start[t] = chunks;
    chunks += int((a.numel[t] + MT_CHUNK - 1) / MT_CHUNK);
  }
  a.chunk_start[a.n_tensors] = chunks;
  if (chunks == 0) return;
  if (a.param_bf16) {
    if (a.grad_bf16) multi_tensor_optim_kernel<__nv_bfloat16, __nv_bfloat16><<<chunks, MT_THREADS, 0, stream>>>(a);
    else multi_tensor_optim_kernel<__nv_bfloat16, float><<<chunks, MT_THREADS, 0, stream>>>(a);
  } else {
    if (a.grad_bf16) multi_tensor_optim_kernel<float, __nv_bfloat16><<<chunks, MT_THREADS, 0, stream>>>(a);
    else multi_tensor_optim_kernel<float, float><<<chunks, MT_THREADS, 0, stream>>>(a);
  }
  RT_LAUNCH_CHECK();
}

}  // namespace rt
