// LayerNorm / RMSNorm forward + backward, bf16 activations, fp32 statistics.
// One warp per row, 16-byte vector loads, rows re-read through L1 instead of staged.
// Backward fuses (a) the optional upstream residual gradient add into dx and (b) the
// gamma/beta gradient reduction (per-CTA partial sums in a scratch buffer, then a small
// column-parallel second stage; no global atomics),
// accumulating straight into the fp32 gradient buffers the fused optimizer consumes.
// Semantics follow the reference's layers (src/nn/normalization.rs:59-99 LayerNorm,
// :587-608,652-701 RMSNorm), which have forward only and no backward.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 t = __bfloat1622float2(h[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 w;
  w.x = pack_bf16x2(f[0], f[1]);
  w.y = pack_bf16x2(f[2], f[3]);
  w.z = pack_bf16x2(f[4], f[5]);
  w.w = pack_bf16x2(f[6], f[7]);
  return w;
}

// RMS = true: y = x * rstd * g (beta ignored, mean = 0).  C % 8 == 0.
// MAXV > 0: the row is cached in registers (C <= 256*MAXV) and read from memory once.
template <bool RMS, int MAXV>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ gamma,
                                const __nv_bfloat16* __restrict__ beta,
                                __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                                float* __restrict__ rstd_out, long long rows, int C, float eps) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
  const int nv = C >> 3;
  uint4 cache[MAXV > 0 ? MAXV : 1];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int vi = 0; vi < (MAXV > 0 ? MAXV : 64); ++vi) {
    const int v = lane + vi * 32;
    if (v >= nv) break;
    const uint4 w = xr[v];
    if (MAXV > 0) cache[vi] = w;
    float f[8];
    unpack8(w, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      s += f[e];
      ss += f[e] * f[e];
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  float mean = RMS ? 0.f : s / C;
  float var;
  if (RMS) {
    var = ss / C;
  } else {
    // second pass for a numerically safe variance
    float sq = 0.f;
#pragma unroll
    for (int vi = 0; vi < (MAXV > 0 ? MAXV : 64); ++vi) {
      const int v = lane + vi * 32;
      if (v >= nv) break;
      float f[8];
      unpack8(MAXV > 0 ? cache[vi] : xr[v], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = f[e] - mean;
        sq += d * d;
      }
    }
    var = warp_sum(sq) / C;
  }
  const float rstd = rsqrtf(var + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + row * C);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const uint4* br = reinterpret_cast<const uint4*>(beta);
#pragma unroll
  for (int vi = 0; vi < (MAXV > 0 ? MAXV : 64); ++vi) {
    const int v = lane + vi * 32;
    if (v >= nv) break;
    float f[8], g[8], o[8];
    unpack8(MAXV > 0 ? cache[vi] : xr[v], f);
    unpack8(gr[v], g);
    if (!RMS && beta) {
      float bb[8];
      unpack8(br[v], bb);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (f[e] - mean) * rstd * g[e] + bb[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (f[e] - mean) * rstd * g[e];
    }
    yr[v] = pack8(o);
  }
}

__device__ __forceinline__ uint4 ld_nc16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// dx = rstd * (g*dy - c1 - xhat*c2) (+ dres);  LayerNorm: c1 = mean(g*dy), c2 = mean(g*dy*xhat)
// RMSNorm: c1 = 0, c2 = mean(g*dy*xhat) with xhat = x*rstd.
// MAXV > 0: per-lane register accumulators for dgamma/dbeta (C <= 256*MAXV); MAXV == 0: shared
// atomics per element.
template <bool RMS, int MAXV>
__global__ void norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ gamma,
                                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                const __nv_bfloat16* __restrict__ dres,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                long long rows, int C) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  // MAXV > 0: one [2][C] slot per warp (plain stores); MAXV == 0: a single [2][C] slot (atomics)
  extern __shared__ float sacc[];
  const int warps = blockDim.x >> 5;
  const int n_slots = MAXV > 0 ? warps : 1;
  float* sdg = sacc;
  float* sdb = sacc + C;
  if (MAXV == 0) {
    for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) sacc[i] = 0.f;
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nv = C >> 3;
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  float adg[MAXV > 0 ? MAXV * 8 : 1], adb[MAXV > 0 ? MAXV * 8 : 1];
#pragma unroll
  for (int i = 0; i < (MAXV > 0 ? MAXV * 8 : 1); ++i) adg[i] = adb[i] = 0.f;
  // MAXV > 0: the row lives in registers (one 16-byte load of x and dy per vector, no second read), and the next row's
  // loads are issued before this row's reductions, so the memory pipe stays busy through the arithmetic.
  // The prefetch costs 8 * MAXV registers: RMSNorm has them (no beta accumulators), LayerNorm at MAXV = 4 would
  // drop to one CTA per SM (168 registers), so LayerNorm loads the row at the top of its own iteration.
  constexpr int NV = MAXV > 0 ? MAXV : 1;
  constexpr bool PREFETCH = MAXV > 0 && RMS;
  constexpr bool CACHE = MAXV > 0 && (RMS || MAXV <= 3);  // LayerNorm at MAXV = 4 re-reads the row (L1) instead
  const long long row_step = (long long)gridDim.x * warps;
  long long row = (long long)blockIdx.x * warps + warp;
  uint4 cx[CACHE ? NV : 1], cd[CACHE ? NV : 1], nx[PREFETCH ? NV : 1], nd[PREFETCH ? NV : 1];
  auto fetch = [&](long long r, auto& fx, auto& fd) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * C);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + r * C);
#pragma unroll
    for (int vi = 0; vi < NV; ++vi) {
      const int v = lane + vi * 32;
      if (v < nv) {
        fx[vi] = ld_nc16(xr + v);
        fd[vi] = ld_nc16(dyr + v);
      }
    }
  };
  if (PREFETCH && row < rows) fetch(row, cx, cd);
  for (; row < rows; row += row_step) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * C);
    if constexpr (PREFETCH) {
      if (row + row_step < rows) fetch(row + row_step, nx, nd);
    } else if constexpr (CACHE) {
      fetch(row, cx, cd);
    }
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float c1 = 0.f, c2 = 0.f;
    if constexpr (CACHE) {
#pragma unroll
      for (int vi = 0; vi < NV; ++vi) {
        const int v = lane + vi * 32;
        if (v < nv) {
          float f[8], d[8], g[8];
          unpack8(cx[vi], f);
          unpack8(cd[vi], d);
          unpack8(gr[v], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float xh = (f[e] - mean) * rstd;
            const float gd = g[e] * d[e];
            c1 += gd;
            c2 += gd * xh;
          }
        }
      }
    } else {
      for (int v = lane; v < nv; v += 32) {
        float f[8], d[8], g[8];
        unpack8(xr[v], f);
        unpack8(dyr[v], d);
        unpack8(gr[v], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (f[e] - mean) * rstd;
          const float gd = g[e] * d[e];
          c1 += gd;
          c2 += gd * xh;
        }
      }
    }
    c1 = RMS ? 0.f : warp_sum(c1) / C;
    c2 = warp_sum(c2) / C;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * C);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * C) : nullptr;
#pragma unroll
    for (int vi = 0; vi < (MAXV > 0 ? MAXV : 64); ++vi) {
      const int v = lane + vi * 32;
      if (v >= nv) break;
      float f[8], d[8], g[8], o[8];
      unpack8(CACHE ? cx[CACHE ? vi : 0] : xr[v], f);
      unpack8(CACHE ? cd[CACHE ? vi : 0] : dyr[v], d);
      unpack8(gr[v], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = (f[e] - mean) * rstd;
        o[e] = rstd * (g[e] * d[e] - c1 - xh * c2);
        if (MAXV > 0) {
          adg[vi * 8 + e] += d[e] * xh;
          if (!RMS) adb[vi * 8 + e] += d[e];
        } else {
          atomicAdd(&sdg[v * 8 + e], d[e] * xh);
          if (!RMS) atomicAdd(&sdb[v * 8 + e], d[e]);
        }
      }
      if (drr) {
        float r[8];
        unpack8(drr[v], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += r[e];
      }
      dxr[v] = pack8(o);
    }
    if constexpr (PREFETCH) {
#pragma unroll
      for (int vi = 0; vi < NV; ++vi) {
        cx[vi] = nx[vi];
        cd[vi] = nd[vi];
      }
    }
  }
  if (MAXV > 0) {
    float* wdg = sacc + (size_t)warp * 2 * C;
    float* wdb = wdg + C;
#pragma unroll
    for (int vi = 0; vi < (MAXV > 0 ? MAXV : 1); ++vi) {
      const int v = lane + vi * 32;
      if (v < nv) {
        float4* g4 = reinterpret_cast<float4*>(wdg + v * 8);
        g4[0] = make_float4(adg[vi * 8 + 0], adg[vi * 8 + 1], adg[vi * 8 + 2], adg[vi * 8 + 3]);
        g4[1] = make_float4(adg[vi * 8 + 4], adg[vi * 8 + 5], adg[vi * 8 + 6], adg[vi * 8 + 7]);
        if (!RMS) {
          float4* b4 = reinterpret_cast<float4*>(wdb + v * 8);
          b4[0] = make_float4(adb[vi * 8 + 0], adb[vi * 8 + 1], adb[vi * 8 + 2], adb[vi * 8 + 3]);
          b4[1] = make_float4(adb[vi * 8 + 4], adb[vi * 8 + 5], adb[vi * 8 + 6], adb[vi * 8 + 7]);
        }
      }
    }
  }
  __syncthreads();
  // per-CTA partial sums: partial[0][cta][C] = dgamma part, partial[1][cta][C] = dbeta part
  float* pg = partial + (long long)blockIdx.x * C;
  float* pb = partial + ((long long)gridDim.x + blockIdx.x) * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float tg = 0.f, tb = 0.f;
    for (int w = 0; w < n_slots; ++w) {
      tg += sacc[(size_t)w * 2 * C + i];
      if (!RMS) tb += sacc[(size_t)w * 2 * C + C + i];
    }
    pg[i] = tg;
    if (!RMS) pb[i] = tb;
  }
}

// Second stage: out[c] += sum over CTAs of partial[.][cta][c].  One CTA covers 32 columns with
// 32 partial-row lanes (coalesced 128-byte reads), combined through shared memory.
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta, int n_part, int C) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  __shared__ float red[32][33];
  const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  const bool is_beta = blockIdx.y == 1;
  float* out = is_beta ? dbeta : dgamma;
  if (out == nullptr) return;
  const float* src = partial + (is_beta ? (long long)n_part * C : 0);
  float acc = 0.f;
  if (c < C)
    for (int g = pl; g < n_part; g += 32) acc += src[(long long)g * C + c];
  red[pl][cl] = acc;
  __syncthreads();
  if (pl == 0 && c < C) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += red[r][cl];
    out[c] += t;
  }
}

void norm_fwd(const NormArgs& a, cudaStream_t stream) {
  RT_CHECK(a.C % 8 == 0, "norm: feature size must be a multiple of 8");
  if (a.rows == 0) return;
  const int wpb = 4;
  const unsigned grid = (unsigned)((a.rows + wpb - 1) / wpb);
  auto x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  auto g = reinterpret_cast<const __nv_bfloat16*>(a.gamma);
  auto b = reinterpret_cast<const __nv_bfloat16*>(a.beta);
  auto y = reinterpret_cast<__nv_bfloat16*>(a.y);
  const bool small = a.C <= 1024;
  if (a.rms) {
    if (small) norm_fwd_kernel<true, 4><<<grid, wpb * 32, 0, stream>>>(x, g, b, y, a.mean, a.rstd, a.rows, a.C, a.eps);
    else norm_fwd_kernel<true, 0><<<grid, wpb * 32, 0, stream>>>(x, g, b, y, a.mean, a.rstd, a.rows, a.C, a.eps);
  } else {
    if (small) norm_fwd_kernel<false, 4><<<grid, wpb * 32, 0, stream>>>(x, g, b, y, a.mean, a.rstd, a.rows, a.C, a.eps);
    else norm_fwd_kernel<false, 0><<<grid, wpb * 32, 0, stream>>>(x, g, b, y, a.mean, a.rstd, a.rows, a.C, a.eps);
  }
  RT_LAUNCH_CHECK();
}

// Wide rows (2048-column multiples up to 8192, e.g. the 4096-wide RMSNorm of an 8B Llama): one CTA per row, every
// thread owns VPT 16-byte vectors of the row for the whole kernel, so gamma and the dgamma / dbeta accumulators sit in
// registers and the CTA's partial sums are written without any cross-thread reduction; only the two row scalars go
// through shared memory (one barrier per row, buffers alternate by row parity).  The next row is prefetched.
template <bool RMS, int VPT>
__global__ void __launch_bounds__(256) norm_bwd_wide_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gamma,
                                                            const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                            const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                                            float* __restrict__ partial, long long rows, int C) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  __shared__ float red[2][2][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint4 gv[VPT];
  float adg[VPT * 8], adb[RMS ? 1 : VPT * 8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) gv[i] = reinterpret_cast<const uint4*>(gamma)[tid + i * 256];
#pragma unroll
  for (int i = 0; i < VPT * 8; ++i) adg[i] = 0.f;
#pragma unroll
  for (int i = 0; i < (RMS ? 1 : VPT * 8); ++i) adb[i] = 0.f;
  uint4 cx[VPT], cd[VPT], nx[VPT], nd[VPT];
  auto fetch = [&](long long r, uint4 (&fx)[VPT], uint4 (&fd)[VPT]) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * C);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + r * C);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      fx[i] = ld_nc16(xr + tid + i * 256);
      fd[i] = ld_nc16(dyr + tid + i * 256);
    }
  };
  long long row = blockIdx.x;
  if (row < rows) fetch(row, cx, cd);
  int par = 0;
  for (; row < rows; row += gridDim.x, par ^= 1) {
    if (row + gridDim.x < rows) fetch(row + gridDim.x, nx, nd);
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float f[8], d[8], g[8];
      unpack8(cx[i], f);
      unpack8(cd[i], d);
      unpack8(gv[i], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = (f[e] - mean) * rstd;
        const float gd = g[e] * d[e];
        c1 += gd;
        c2 += gd * xh;
      }
    }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if (lane == 0) {
      red[par][0][warp] = c1;
      red[par][1][warp] = c2;
    }
    __syncthreads();
    c1 = c2 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      c1 += red[par][0][w];
      c2 += red[par][1][w];
    }
    c1 = RMS ? 0.f : c1 / C;
    c2 = c2 / C;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * C);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * C) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float f[8], d[8], g[8], o[8];
      unpack8(cx[i], f);
      unpack8(cd[i], d);
      unpack8(gv[i], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = (f[e] - mean) * rstd;
        o[e] = rstd * (g[e] * d[e] - c1 - xh * c2);
        adg[i * 8 + e] += d[e] * xh;
        if (!RMS) adb[i * 8 + e] += d[e];
      }
      if (drr) {
        float r[8];
        unpack8(drr[tid + i * 256], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += r[e];
      }
      dxr[tid + i * 256] = pack8(o);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      cx[i] = nx[i];
      cd[i] = nd[i];
    }
  }
  float* pg = partial + (long long)blockIdx.x * C;
  float* pb = partial + ((long long)gridDim.x + blockIdx.x) * C;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c0 = (tid + i * 256) * 8;
    float4* g4 = reinterpret_cast<float4*>(pg + c0);
    g4[0] = make_float4(adg[i * 8 + 0], adg[i * 8 + 1], adg[i * 8 + 2], adg[i * 8 + 3]);
    g4[1] = make_float4(adg[i * 8 + 4], adg[i * 8 + 5], adg[i * 8 + 6], adg[i * 8 + 7]);
    if (!RMS) {
      float4* b4 = reinterpret_cast<float4*>(pb + c0);
      b4[0] = make_float4(adb[i * 8 + 0], adb[i * 8 + 1], adb[i * 8 + 2], adb[i * 8 + 3]);
      b4[1] = make_float4(adb[i * 8 + 4], adb[i * 8 + 5], adb[i * 8 + 6], adb[i * 8 + 7]);
    }
  }
}

template <bool RMS, int VPT>
static void launch_norm_bwd_wide(const NormArgs& a, unsigned grid, cudaStream_t stream) {
  norm_bwd_wide_kernel<RMS, VPT><<<grid, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(a.dy), reinterpret_cast<const __nv_bfloat16*>(a.x),
      reinterpret_cast<const __nv_bfloat16*>(a.gamma), a.mean, a.rstd, reinterpret_cast<const __nv_bfloat16*>(a.dres),
      reinterpret_cast<__nv_bfloat16*>(a.dx), a.partial, a.rows, a.C);
  RT_LAUNCH_CHECK();
}

template <bool RMS, int MAXV>
static void launch_norm_bwd(const NormArgs& a, unsigned grid, int threads, size_t smem,
                            cudaStream_t stream) {
  auto kern = norm_bwd_kernel<RMS, MAXV>;
  if (smem > 48 * 1024)
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, threads, smem, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(a.dy), reinterpret_cast<const __nv_bfloat16*>(a.x),
      reinterpret_cast<const __nv_bfloat16*>(a.gamma), a.mean, a.rstd,
      reinterpret_cast<const __nv_bfloat16*>(a.dres), reinterpret_cast<__nv_bfloat16*>(a.dx),
      a.partial, a.rows, a.C);
  RT_LAUNCH_CHECK();
}

int norm_bwd_num_partials(long long rows, int sm_count) {
  const int warps = 8;
  const long long want = (rows + warps - 1) / warps;
  return (int)std::max<long long>(1, std::min<long long>(want, 2LL * sm_count));
}

// Stage 1 (dx and the per-CTA partial sums); with a null `reduce_stream` the second stage follows on `stream`, otherwise
// the caller runs norm_bwd_reduce itself (on another stream, after an event) so that dx is not held up by it.
void norm_bwd_stage1(const NormArgs& a, cudaStream_t stream, const cudaStream_t* reduce_stream) {
  RT_CHECK(a.C % 8 == 0, "norm: feature size must be a multiple of 8");
  RT_CHECK(a.C <= 16384, "norm backward: feature size above 16384 not supported");
  if (a.rows == 0) return;
  RT_CHECK(a.partial != nullptr && a.n_partial >= 1, "norm backward: scratch for partial sums missing");
  const int threads = 256;
  const unsigned grid = (unsigned)a.n_partial;
  const bool small = a.C <= 1024;
  const size_t smem = sizeof(float) * 2 * a.C * (small ? threads / 32 : 1);
  const int vpt = (!small && a.C % 2048 == 0 && a.C <= 8192) ? a.C / 2048 : 0;  // wide rows: one CTA per row
  const int maxv = small ? (a.C + 255) / 256 : 0;  // 16-byte vectors per lane
#define RT_NORM_BWD(R)                                                        \
  do {                                                                        \
    if (maxv == 1) launch_norm_bwd<R, 1>(a, grid, threads, smem, stream);     \
    else if (maxv == 2) launch_norm_bwd<R, 2>(a, grid, threads, smem, stream); \
    else if (maxv == 3) launch_norm_bwd<R, 3>(a, grid, threads, smem, stream); \
    else if (maxv == 4) launch_norm_bwd<R, 4>(a, grid, threads, smem, stream); \
    else launch_norm_bwd<R, 0>(a, grid, threads, smem, stream);               \
  } while (0)
  if (vpt == 1 || vpt == 2 || vpt == 4) {
    if (a.rms) {
      if (vpt == 1) launch_norm_bwd_wide<true, 1>(a, grid, stream);
      else if (vpt == 2) launch_norm_bwd_wide<true, 2>(a, grid, stream);
      else launch_norm_bwd_wide<true, 4>(a, grid, stream);
    } else {
      if (vpt == 1) launch_norm_bwd_wide<false, 1>(a, grid, stream);
      else if (vpt == 2) launch_norm_bwd_wide<false, 2>(a, grid, stream);
      else launch_norm_bwd_wide<false, 4>(a, grid, stream);
    }
  } else if (a.rms) RT_NORM_BWD(true);
  else RT_NORM_BWD(false);
#undef RT_NORM_BWD
  if (reduce_stream == nullptr) norm_bwd_reduce(a, stream);
}

void norm_bwd_reduce(const NormArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return;
  if (a.dgamma != nullptr || (!a.rms && a.dbeta != nullptr)) {
    dim3 g2((a.C + 31) / 32, a.rms ? 1 : 2);
    norm_bwd_reduce_kernel<<<g2, 1024, 0, stream>>>(a.partial, a.dgamma, a.dbeta, a.n_partial, a.C);
    RT_LAUNCH_CHECK();
  }
}

void norm_bwd(const NormArgs& a, cudaStream_t stream) { norm_bwd_stage1(a, stream, nullptr); }

}  // namespace rt
