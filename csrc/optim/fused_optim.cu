// Fused flat-buffer optimizer step: one pass over fp32 master weights + moments + gradients
// that applies the gradient scale, the update rule, refreshes the bf16 compute copy of the
// parameters and zeroes the gradient for the next step (read 16 B, write 18 B per parameter).
// Update rules mirror the reference's per-tensor host loops: AdamW decoupled decay
// p *= (1 - lr*wd) (src/optim/adamw.rs:159-163), Adam with L2-in-gradient decay
// (src/optim/mod.rs:218-404), SGD with momentum/dampening/nesterov/L2 decay
// (src/optim/mod.rs:82-214).  The step counter is per optimizer step, not per tensor.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

__device__ __forceinline__ void optim_update(const OptimArgs& a, float& p, float& g, float& m,
                                             float& v) {
  g *= a.grad_scale;
  if (a.mode == OPT_ADAMW || a.mode == OPT_ADAM) {
    if (a.mode == OPT_ADAM) g += a.weight_decay * p;
    m = a.beta1 * m + (1.f - a.beta1) * g;
    v = a.beta2 * v + (1.f - a.beta2) * g * g;
    const float mhat = m / a.bias_corr1;
    const float vhat = v / a.bias_corr2;
    if (a.mode == OPT_ADAMW) p *= (1.f - a.lr * a.weight_decay);
    p -= a.lr * mhat / (sqrtf(vhat) + a.eps);
  } else {  // OPT_SGD: beta1 = momentum, beta2 = dampening, first_step => buffer = g
    g += a.weight_decay * p;
    float d = g;
    if (a.beta1 != 0.f) {
      m = a.first_step ? g : (a.beta1 * m + (1.f - a.beta2) * g);
      d = a.nesterov ? (g + a.beta1 * m) : m;
    }
    p -= a.lr * d;
  }
}

__global__ void fused_optim_kernel(const OptimArgs a) {
  const long long n4 = a.n >> 2;
  float4* P = reinterpret_cast<float4*>(a.master);
  float4* G = reinterpret_cast<float4*>(a.grad);
  float4* M = reinterpret_cast<float4*>(a.m);
  float4* V = reinterpret_cast<float4*>(a.v);
  const bool has_v = a.v != nullptr;
  const bool has_m = a.m != nullptr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = P[i], g = G[i];
    float4 m = has_m ? M[i] : make_float4(0, 0, 0, 0);
    float4 v = has_v ? V[i] : make_float4(0, 0, 0, 0);
    optim_update(a, p.x, g.x, m.x, v.x);
    optim_update(a, p.y, g.y, m.y, v.y);
    optim_update(a, p.z, g.z, m.z, v.z);
    optim_update(a, p.w, g.w, m.w, v.w);
    P[i] = p;
    if (has_m) M[i] = m;
    if (has_v) V[i] = v;
    if (a.zero_grad) G[i] = make_float4(0, 0, 0, 0);
    if (a.param_lp) {
      uint2 w;
      w.x = pack_bf16x2(p.x, p.y);
      w.y = pack_bf16x2(p.z, p.w);
      reinterpret_cast<uint2*>(a.param_lp)[i] = w;
    }
  }
  // tail (n % 4)
  if (blockIdx.x == 0 && threadIdx.x < (a.n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    float p = a.master[i], g = a.grad[i];
    float m = has_m ? a.m[i] : 0.f, v = has_v ? a.v[i] : 0.f;
    optim_update(a, p, g, m, v);
    a.master[i] = p;
    if (has_m) a.m[i] = m;
    if (has_v) a.v[i] = v;
    if (a.zero_grad) a.grad[i] = 0.f;
    if (a.param_lp) reinterpret_cast<__nv_bfloat16*>(a.param_lp)[i] = __float2bfloat16(p);
  }
}

void fused_optim_step(const OptimArgs& a, cudaStream_t stream) {
  if (a.n == 0) return;
  RT_CHECK((reinterpret_cast<uintptr_t>(a.master) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(a.grad) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(a.m) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(a.v) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(a.param_lp) & 7) == 0,
           "fused_optim_step: buffers must be 16-byte aligned");
  const int threads = 256;
  const long long n4 = std::max<long long>(1, a.n >> 2);
  const int grid = (int)std::min<long long>((n4 + threads - 1) / threads, 8LL * sm_count(current_device()));
  fused_optim_kernel<<<grid, threads, 0, stream>>>(a);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
