// Llama block glue kernels (bf16): rotary embedding fused with the q / k / v split, and SwiGLU.
//
//   rope_split   qkv [rows][(H + 2 Hkv) D] (one GEMM output) -> q [rows][H][D], k [rows][Hkv][D], v [rows][Hkv][D],
//                rotating the pairs (i, i + D/2) of q and k by the angle of the row's position (row mod T); backward
//                rotates dq, dk by the opposite angle and packs dq | dk | dv back into d(qkv).  One pass each way
//                instead of slice / multiply / concatenate chains over three tensors.
//   swiglu       gu [rows][2 F] (gate | up) -> act = silu(gate) * up; backward writes d(gate) | d(up) from d(act), gu.
//
// Angles come from cos / sin tables [T][D/2] (fp32).  A thread handles 8 consecutive elements of the first half of a
// head and their partners in the second half (two 16-byte loads, two stores).
// Reference: SwiGLU is src/nn/activation.rs:378-419; the reference has no rotary embedding (its attention,
// example-cli/src/model/architectures/attention.rs, applies none), the rotation here is the Llama convention.
#include <cuda_bf16.h>

#include <algorithm>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// backward = false: packed -> (q, k, v) with rotation; true: (dq, dk, dv) -> packed with the inverse rotation.
template <bool BWD>
__global__ void __launch_bounds__(256) rope_split_kernel(__nv_bfloat16* __restrict__ packed, __nv_bfloat16* __restrict__ q,
                                                         __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                                                         const float* __restrict__ cs, const float* __restrict__ sn, long long rows,
                                                         int T, int H, int Hkv, int D) {
  const int half = D / 2, hv = half / 8;                 // 8-element vectors per half head
  const int heads = H + 2 * Hkv;
  const long long total = rows * heads * hv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(t % hv) * 8;
    long long r = t / hv;
    const int head = (int)(r % heads);
    r /= heads;
    const int pos = (int)(r % T);
    __nv_bfloat16* pk = packed + (r * heads + head) * D;
    __nv_bfloat16* dst;
    if (head < H) dst = q + (r * H + head) * D;
    else if (head < H + Hkv) dst = k + (r * Hkv + (head - H)) * D;
    else dst = v + (r * Hkv + (head - H - Hkv)) * D;
    __nv_bfloat16* src = BWD ? dst : pk;
    __nv_bfloat16* out = BWD ? pk : dst;
    float a[8], b[8];
    ld8(src + i, a);
    ld8(src + half + i, b);
    if (head < H + Hkv) {
      const float4 c0 = *reinterpret_cast<const float4*>(cs + (long long)pos * half + i);
      const float4 c1 = *reinterpret_cast<const float4*>(cs + (long long)pos * half + i + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sn + (long long)pos * half + i);
      const float4 s1 = *reinterpret_cast<const float4*>(sn + (long long)pos * half + i + 4);
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float sg = BWD ? -s[e] : s[e];
        const float x0 = a[e] * c[e] - b[e] * sg, x1 = a[e] * sg + b[e] * c[e];
        a[e] = x0;
        b[e] = x1;
      }
    }
    st8(out + i, a);
    st8(out + half + i, b);
  }
}

__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                                         long long rows, int F) {
  const int fv = F / 8;
  const long long total = rows * fv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / fv;
    const int j = (int)(t % fv) * 8;
    float g[8], u[8];
    ld8(gu + r * 2 * F + j, g);
    ld8(gu + r * 2 * F + F + j, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    st8(act + r * F + j, g);
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                                         __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const int fv = F / 8;
  const long long total = rows * fv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / fv;
    const int j = (int)(t % fv) * 8;
    float g[8], u[8], d[8];
    ld8(gu + r * 2 * F + j, g);
    ld8(gu + r * 2 * F + F + j, u);
    ld8(dact + r * F + j, d);
    float dg[8], du[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float s = 1.f / (1.f + __expf(-g[e]));
      const float silu = g[e] * s;
      du[e] = d[e] * silu;
      dg[e] = d[e] * u[e] * (s + silu * (1.f - s));
    }
    st8(dgu + r * 2 * F + j, dg);
    st8(dgu + r * 2 * F + F + j, du);
  }
}

int grid_sz(long long work, int device) { return (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, 8LL * sm_count(device))); }

}  // namespace

void rope_split(void* packed, void* q, void* k, void* v, const float* cos_t, const float* sin_t, long long rows, int T, int H, int Hkv,
                int D, bool backward, cudaStream_t s) {
  RT_CHECK(D % 16 == 0 && T >= 1 && H >= 1 && Hkv >= 1, "rope_split: head dim must be a multiple of 16");
  if (rows == 0) return;
  const int grid = grid_sz(rows * (H + 2 * Hkv) * (D / 16), current_device());
  auto pk = reinterpret_cast<__nv_bfloat16*>(packed);
  auto pq = reinterpret_cast<__nv_bfloat16*>(q);
  auto pkk = reinterpret_cast<__nv_bfloat16*>(k);
  auto pv = reinterpret_cast<__nv_bfloat16*>(v);
  if (backward) rope_split_kernel<true><<<grid, 256, 0, s>>>(pk, pq, pkk, pv, cos_t, sin_t, rows, T, H, Hkv, D);
  else rope_split_kernel<false><<<grid, 256, 0, s>>>(pk, pq, pkk, pv, cos_t, sin_t, rows, T, H, Hkv, D);
  RT_LAUNCH_CHECK();
}

void swiglu(const void* gu, const void* dact, void* out, long long rows, int F, bool backward, cudaStream_t s) {
  RT_CHECK(F % 8 == 0, "swiglu: hidden size must be a multiple of 8");
  if (rows == 0 || F == 0) return;
  const int grid = grid_sz(rows * (F / 8), current_device());
  if (backward)
    swiglu_bwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<const __nv_bfloat16*>(dact),
                                           reinterpret_cast<__nv_bfloat16*>(out), rows, F);
  else swiglu_fwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<__nv_bfloat16*>(out), rows, F);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
