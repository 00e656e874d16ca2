// Decode-step projections as one kernel each: RMSNorm prologue + dequant-fused Q4_0 / Q8_0 GEMV + epilogue.
//
//   h[m][k]  = x[m][k] * rsqrt(mean_k x[m][k]^2 + eps) * norm_w[k]     (optional prologue)
//   t[m][n]  = sum_k dequant(W)[n][k] * h[m][k]
//   y[m][n]  = t[m][n] (+ residual[m][n])                               (plain epilogue), or
//   y[m][i]  = silu(t[m][i]) * t[m][ff + i]                             (SwiGLU epilogue over a [gate; up] matrix), or
//   y[m]     = [rope(q); rope(k); v] with k and v also appended to the KV cache   (rotary epilogue over [q; k; v])
//
// for M <= 4 activation rows.  A decode step of a Llama layer is then four of these (qkv, wo, gate/up, down) plus
// the rotary / cache / attention kernels, instead of four GEMVs, two RMSNorm and one SwiGLU launch.
//
// Arithmetic: the staged activations are quantised to int8 per 32-element block (scale = max |h| / 127, the Q8_1
// scheme llama.cpp multiplies its quantised weights with), so a block's dot product is eight dp4a instructions on
// the raw nibbles (masked in place, no conversion to fp16) instead of ~50 integer / half2 instructions:
//   sum_k (q_k - 8) d_w * xq_k d_x = d_w d_x (sum_k q_k xq_k - 8 sum_k xq_k)
// with the second sum computed once per block while staging.  The fp16-activation GEMV spends ~3.6 instructions per
// weight byte on the expansion and levels off near 2.9 TB/s; this one is bound by the weight stream.
//
// Work split: the CTA first stages the (normalised, quantised) activation rows in shared memory; the weights' first
// loads are issued before that, and before the wait on the previous kernel, since weights never depend on it.  A warp
// owns four output rows (SwiGLU: two gate rows and their two up rows) over the whole K; lane l walks blocks l,
// l + 32, ... with the raw blocks of the next two steps already in flight (three block-steps of 4 rows x 16 bytes
// per lane).  No shared-memory reduction across warps: one shuffle reduction per row finishes it.
// Device weight layout: see q_gemv.cu.  The reference runs these projections as scalar host loops over f64
// (example-cli/src/model/architectures/attention.rs:233-303, model/inference.rs:135-192).
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "q_expand.cuh"

namespace rt {

constexpr int QF_R = 4;       // rows per warp
constexpr int QF_WARPS = 8;   // warps per CTA
// block-steps of the per-warp shared-memory ring (one being multiplied, the others in flight by cp.async): Q8_0
// blocks are twice as large
template <bool Q8>
constexpr int qf_depth() { return Q8 ? 3 : 4; }

// Asks the L2 for this CTA's share of [p, p + bytes) in 16 KB pieces (a hint: nothing waits for it).
__device__ __forceinline__ void prefetch_l2_slice(const uint8_t* p, long long bytes, int cta, int n_cta) {
  if (p == nullptr || bytes <= 0) return;
  constexpr long long PIECE = 16384;
  const long long pieces = (bytes + PIECE - 1) / PIECE;
  for (long long i = cta; i < pieces; i += n_cta) {
    const long long off = i * PIECE;
    const unsigned sz = unsigned(min(PIECE, bytes - off)) & ~15u;
    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(sz) : "memory");
  }
}

template <bool Q8>
struct QfRaw {
  uint4 v[Q8 ? 2 : 1];
};

// Rotary epilogue of the fused q | k | v projection (pairs (2i, 2i + 1) of a head, as GGUF Llama weights expect): q and
// k rows are rotated by the token's position, k and v rows are also appended to the KV cache.
struct QfRope {
  const int* pos;   // [M] position of each token in its sequence
  const int* seq;   // [M] sequence (cache batch) index of each token
  __half* cache_k;  // [n_seq][Hkv][T_max][D]
  __half* cache_v;
  int H, Hkv, D, T_max, n_seq;
  float log2_theta;
  int* status;
};

// EPI: 0 = plain / residual, 1 = SwiGLU over [gate; up] rows, 2 = rotary + KV-cache append over [q; k; v] rows
template <bool Q8, int M, int EPI>
__global__ void __launch_bounds__(QF_WARPS * 32, 2) q_gemv_fused_kernel(const void* __restrict__ qs, const __half* __restrict__ scales,
                                                                     const __half* __restrict__ x, long long ldx,
                                                                     const __half* __restrict__ norm_w, float eps,
                                                                     __half* __restrict__ y, long long ldy,
                                                                     const __half* __restrict__ residual, long long ldr,
                                                                     int N, int K, const uint8_t* __restrict__ pf0,
                                                                     long long pf0_bytes, const uint8_t* __restrict__ pf1,
                                                                     long long pf1_bytes, const QfRope rope) {
  constexpr bool SWIGLU = EPI == 1, ROPE = EPI == 2;
  extern __shared__ __align__(16) uint8_t qf_smem[];
  __shared__ float red[M][QF_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int QF_DEPTH = qf_depth<Q8>();
  const int nb = K >> 5;  // 32-weight blocks per row
  const int ff = N >> 1;  // SWIGLU: rows [0, ff) are the gate, [ff, N) the up projection
  const int out_n = SWIGLU ? ff : N;
  // The grid is what is resident at once, so the activation staging below is paid once per SM slot.  Every warp of
  // the grid owns a contiguous, equally long range of output rows (SWIGLU: gate/up pairs) and walks it in items of
  // up to 4 rows (2 pairs).
  constexpr int PER_ITEM = SWIGLU ? QF_R / 2 : QF_R;
  const long long all_warps = (long long)gridDim.x * QF_WARPS;
  const long long gw = (long long)blockIdx.x * QF_WARPS + warp;
  // ROPE: ranges in whole items of four rows, so that a rotation pair never straddles two warps (N % 4 == 0)
  const int u_begin = ROPE ? 4 * int((out_n >> 2) * gw / all_warps) : int(out_n * gw / all_warps);
  const int u_end = ROPE ? 4 * int((out_n >> 2) * (gw + 1) / all_warps) : int(out_n * (gw + 1) / all_warps);
  const int spi = (nb + 31) >> 5;  // block-steps per item: lane l takes block l + 32 k in step k

  // The weight stream of a warp is one sequence of block-steps over all its items; the loads run QF_DEPTH steps
  // ahead of the arithmetic and never drain at an item boundary.  (fu, fk): item start and step of the next fetch.
  int fu = u_begin, fk = 0;
  auto row_active = [&](int r, int n_act) { return SWIGLU ? (r & 1) < n_act : r < n_act; };
  // Per-warp ring in shared memory behind the activations: slot s holds, for each of the 4 rows, the lanes' raw
  // blocks (16 / 32 bytes per lane) and their scales (2 bytes per lane, copied 4 bytes at a time by the even lanes).
  // cp.async groups, not registers and scoreboards, track what is in flight, so all QF_DEPTH steps really overlap.
  constexpr int RAW_B = Q8 ? 32 : 16;
  constexpr int SLOT_BYTES = QF_R * 32 * RAW_B + QF_R * 32 * 2;
  uint8_t* ring_base = qf_smem + (((size_t)M * (K + nb * 8) + 15) & ~size_t(15)) + (size_t)warp * QF_DEPTH * SLOT_BYTES;
  auto fetch = [&](int slot) {
    if (fu < u_end) {
      const int b = lane + (fk << 5);
      const int n_act = min(PER_ITEM, u_end - fu);
      if (b < nb) {
        uint8_t* sl = ring_base + slot * SLOT_BYTES;
#pragma unroll
        for (int r = 0; r < QF_R; ++r) {
          if (row_active(r, n_act)) {
            const int row = SWIGLU ? ((r < 2) ? 0 : ff) + fu + (r & 1) : fu + r;
            const long long off = (long long)row * nb + b;   // N * K / 32 < 2^31 is checked on the host
            const uint8_t* src = reinterpret_cast<const uint8_t*>(qs) + off * RAW_B;
            const uint32_t dst = smem_u32(sl + (r * 32 + lane) * RAW_B);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            if (Q8) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16), "l"(src + 16) : "memory");
            if ((lane & 1) == 0)  // nb is even: blocks b and b + 1 are both in range and the pair is 4-byte aligned
              asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(sl + QF_R * 32 * RAW_B + (r * 32 + lane) * 2)),
                           "l"(scales + off)
                           : "memory");
          }
        }
      }
      if (++fk == spi) {
        fk = 0;
        fu += PER_ITEM;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // every call commits (possibly empty) so group counts stay uniform
  };

  pdl_launch_dependents();
#pragma unroll
  for (int s = 0; s < QF_DEPTH; ++s) fetch(s);
  // ---- pull the NEXT projection's weights towards L2 while this one runs (each CTA asks for its share)
  if (threadIdx.x == 0) {
    prefetch_l2_slice(pf0, pf0_bytes, blockIdx.x, gridDim.x);
    prefetch_l2_slice(pf1, pf1_bytes, blockIdx.x, gridDim.x);
  }
  pdl_wait();

  // ---- stage the activations in one pass: x * norm_w quantised to int8 per block (eight lanes share a block), the
  // sum of squares of x on the side; rsqrt(mean + eps) is a per-row scalar and is applied to the finished sums.
  int8_t* xq = reinterpret_cast<int8_t*>(qf_smem);                          // [M][K]
  float* xd = reinterpret_cast<float*>(qf_smem + (size_t)M * K);            // [M][nb]
  int* xs8 = reinterpret_cast<int*>(xd + (size_t)M * nb);                   // [M][nb]
  float ssq[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    ssq[m] = 0.f;
    const uint2* xr = reinterpret_cast<const uint2*>(x + m * ldx);          // 4 halves per load
    for (int base = 0; base < (K >> 2); base += blockDim.x) {              // whole warps take part in the shuffles
      const int i = base + threadIdx.x;
      const bool valid = i < (K >> 2);                                       // K % 32 == 0: 8-lane groups are whole
      const uint2 v = valid ? __ldg(xr + i) : make_uint2(0u, 0u);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
      float f[4];
      {
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
        f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y;
      }
      if (norm_w != nullptr && valid) {
        ssq[m] += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
        const uint2 g = __ldg(reinterpret_cast<const uint2*>(norm_w) + i);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        const float2 g0 = __half22float2(gh[0]), g1 = __half22float2(gh[1]);
        f[0] *= g0.x; f[1] *= g0.y; f[2] *= g1.x; f[3] *= g1.y;
      }
      float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float inv = amax > 0.f ? 127.f / amax : 0.f;
      int qv[4], qsum = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qv[e] = __float2int_rn(f[e] * inv);
        qsum += qv[e];
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
      if (!valid) continue;
      const int blk = i >> 3, j4 = (i & 7) * 4;                              // elements j4 .. j4 + 3 of block blk
      uint32_t packed = uint32_t(uint8_t(qv[0])) | (uint32_t(uint8_t(qv[1])) << 8) | (uint32_t(uint8_t(qv[2])) << 16) |
                        (uint32_t(uint8_t(qv[3])) << 24);
      if (Q8) {
        *reinterpret_cast<uint32_t*>(xq + (size_t)m * K + blk * 32 + j4) = packed;
      } else {
        // Q4_0 word w = el / 8 holds weights 8w .. 8w + 7; its low-nibble bytes are weights (0, 4, 1, 5) and its
        // high-nibble bytes weights (2, 6, 3, 7): bytes [8w, 8w + 4) pair with the former, [8w + 4, 8w + 8) with the latter
        int8_t* dstb = xq + (size_t)m * K + blk * 32;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int el = j4 + e, p = el & 7;
          dstb[(el & ~7) | ((p & 1) << 1) | (p >> 2) | ((p & 2) << 1)] = (int8_t)qv[e];
        }
      }
      if ((i & 7) == 0) {
        xd[m * nb + blk] = amax / 127.f;
        xs8[m * nb + blk] = 8 * qsum;
      }
    }
    if (norm_w != nullptr) {
      ssq[m] = warp_sum_f(ssq[m]);
      if (lane == 0) red[m][warp] = ssq[m];
    }
  }
  __syncthreads();
  float rs[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    rs[m] = 1.f;
    if (norm_w != nullptr) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < QF_WARPS; ++w) t += red[m][w];
      rs[m] = rsqrtf(t / K + eps);
    }
  }

  float acc[QF_R][M];
#pragma unroll
  for (int r = 0; r < QF_R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  int cu = u_begin, ck = 0;  // item start and step of the arithmetic
  while (cu < u_end) {
#pragma unroll
    for (int s = 0; s < QF_DEPTH; ++s) {   // slot s of the ring holds the step that is s ahead at the loop top
      if (cu < u_end) {
        const int bb = lane + (ck << 5);
        const int n_act = min(PER_ITEM, u_end - cu);
        // take the slot's registers, then refill the slot QF_DEPTH steps ahead
        QfRaw<Q8> cur[QF_R];
        __half dcur[QF_R];
        asm volatile("cp.async.wait_group %0;" ::"n"(QF_DEPTH - 1) : "memory");  // the oldest step has landed
        __syncwarp();                                                            // ... for every lane (scales are shared by pairs)
        {
          const uint8_t* sl = ring_base + s * SLOT_BYTES;
#pragma unroll
          for (int r = 0; r < QF_R; ++r) {
            if (row_active(r, n_act) && bb < nb) {
              cur[r].v[0] = *reinterpret_cast<const uint4*>(sl + (r * 32 + lane) * RAW_B);
              if (Q8) cur[r].v[Q8 ? 1 : 0] = *reinterpret_cast<const uint4*>(sl + (r * 32 + lane) * RAW_B + 16);
              dcur[r] = *reinterpret_cast<const __half*>(sl + QF_R * 32 * RAW_B + (r * 32 + lane) * 2);
            }
          }
        }
        __syncwarp();  // the slot is read by all lanes before anyone refills it
        fetch(s);
        if (bb < nb) {
          uint4 xa[M][2];
          float dx[M];
          int xs[M];
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xq + (size_t)m * K + (bb << 5));
            xa[m][0] = xp[0];
            xa[m][1] = xp[1];
            dx[m] = xd[m * nb + bb];
            xs[m] = xs8[m * nb + bb];
          }
#pragma unroll
          for (int r = 0; r < QF_R; ++r) {
            if (!row_active(r, n_act)) continue;  // warp-uniform
            const float dw = __half2float(dcur[r]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const int xw[8] = {(int)xa[m][0].x, (int)xa[m][0].y, (int)xa[m][0].z, (int)xa[m][0].w,
                                 (int)xa[m][1].x, (int)xa[m][1].y, (int)xa[m][1].z, (int)xa[m][1].w};
              int isum = 0;
              if (Q8) {
                const uint32_t ww[8] = {cur[r].v[0].x, cur[r].v[0].y, cur[r].v[0].z, cur[r].v[0].w,
                                        cur[r].v[Q8 ? 1 : 0].x, cur[r].v[Q8 ? 1 : 0].y, cur[r].v[Q8 ? 1 : 0].z, cur[r].v[Q8 ? 1 : 0].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) isum = __dp4a((int)ww[i], xw[i], isum);
                acc[r][m] = fmaf(dw * dx[m], (float)isum, acc[r][m]);
              } else {
                const uint32_t ww[4] = {cur[r].v[0].x, cur[r].v[0].y, cur[r].v[0].z, cur[r].v[0].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  isum = __dp4a((int)(ww[i] & 0x0F0F0F0Fu), xw[2 * i], isum);
                  isum = __dp4a((int)((ww[i] >> 4) & 0x0F0F0F0Fu), xw[2 * i + 1], isum);
                }
                acc[r][m] = fmaf(dw * dx[m], (float)(isum - xs[m]), acc[r][m]);
              }
            }
          }
        }
        if (++ck == spi) {
          // ---- the item is complete: reduce over the lanes, epilogue, start the next item
#pragma unroll
          for (int r = 0; r < QF_R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = warp_sum_f(acc[r][m]) * rs[m];
          if (lane == 0) {
            if (SWIGLU) {
#pragma unroll
              for (int j2 = 0; j2 < 2; ++j2) {
                if (j2 >= n_act) continue;
                const int n = cu + j2;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                  // gate and up rounded to fp16 first, as the two-kernel path stores them
                  const float g = __half2float(__float2half(acc[j2][m])), up = __half2float(__float2half(acc[2 + j2][m]));
                  y[m * ldy + n] = __float2half(g / (1.f + __expf(-g)) * up);
                }
              }
            } else if (ROPE) {
#pragma unroll
              for (int j2 = 0; j2 < 2; ++j2) {
                const int n = cu + 2 * j2;                 // rows n, n + 1: one rotation pair (items are whole here)
                const int qk_end = (rope.H + rope.Hkv) * rope.D, q_end = rope.H * rope.D;
                const int d0 = n % rope.D;                 // even index inside the head
                const float inv_freq = exp2f(-(float)d0 / (float)rope.D * rope.log2_theta);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                  const int p = rope.pos[m], sq = rope.seq[m];
                  const bool ok = p >= 0 && p < rope.T_max && sq >= 0 && sq < rope.n_seq;
                  if (!ok) atomicCAS(rope.status, 0, RT_ERR_BOUNDS);   // reported; the cache is not touched
                  // rounded to fp16 first, as the separate rotary kernel reads the projection's fp16 output
                  const float a = __half2float(__float2half(acc[2 * j2][m])), b = __half2float(__float2half(acc[2 * j2 + 1][m]));
                  __half ra = __float2half(a), rb = __float2half(b);
                  if (n < qk_end) {
                    float sn, cs;
                    sincosf((float)p * inv_freq, &sn, &cs);
                    ra = __float2half(a * cs - b * sn);
                    rb = __float2half(a * sn + b * cs);
                  }
                  y[m * ldy + n] = ra;
                  y[m * ldy + n + 1] = rb;
                  if (n >= q_end && ok) {
                    const bool is_k = n < qk_end;
                    const int hk = (n - (is_k ? q_end : qk_end)) / rope.D;
                    __half* dst = (is_k ? rope.cache_k : rope.cache_v) + (((long long)sq * rope.Hkv + hk) * rope.T_max + p) * rope.D + d0;
                    dst[0] = ra;
                    dst[1] = rb;
                  }
                }
              }
            } else {
#pragma unroll
              for (int r = 0; r < QF_R; ++r) {
                if (r >= n_act) continue;
                const int n = cu + r;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                  float v = acc[r][m];
                  if (residual) v += __half2float(residual[m * ldr + n]);
                  y[m * ldy + n] = __float2half(v);
                }
              }
            }
          }
#pragma unroll
          for (int r = 0; r < QF_R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
          ck = 0;
          cu += PER_ITEM;
        }
      }
    }
  }
}

template <bool Q8, int M, int EPI>
static void launch_fused(const QGemvFusedArgs& a, cudaStream_t s) {
  constexpr bool SWIGLU = EPI == 1;
  auto kern = q_gemv_fused_kernel<Q8, M, EPI>;
  QfRope rope{};
  if (EPI == 2) {
    rope.pos = a.rope_pos;
    rope.seq = a.rope_seq;
    rope.cache_k = reinterpret_cast<__half*>(a.cache_k);
    rope.cache_v = reinterpret_cast<__half*>(a.cache_v);
    rope.H = a.rope_H;
    rope.Hkv = a.rope_Hkv;
    rope.D = a.rope_D;
    rope.T_max = a.rope_T_max;
    rope.n_seq = a.rope_n_seq;
    rope.log2_theta = log2f(a.rope_theta);
    rope.status = status_word(current_device());
  }
  constexpr int RAW_B = Q8 ? 32 : 16;
  // int8 activations + per-block scale and sum, then the warps' cp.async rings
  const size_t smem = ((size_t(M) * (a.K + (a.K / 32) * 8) + 15) & ~size_t(15)) +
                      size_t(QF_WARPS) * qf_depth<Q8>() * (QF_R * 32 * RAW_B + QF_R * 32 * 2);
  static size_t configured[64] = {0};
  const int device = current_device();
  if (smem > 48 * 1024 && configured[device] < smem) {  // the attribute is per kernel instance and per device
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    configured[device] = smem;
  }
  const int outs = SWIGLU ? a.N / 2 : a.N;
  const int per_cta = QF_WARPS * (SWIGLU ? QF_R / 2 : QF_R);
  int per_sm = 1;  // CTAs of this instance and shared-memory size that fit an SM at once
  RT_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, QF_WARPS * 32, smem));
  // RUSTORCH_QF_CTAS_PER_SM caps the CTAs per SM (tuning; one per SM leaves room for the next kernel's CTA under
  // programmatic dependent launch, which measured slower than filling the SM).
  static const int cap = [] {
    const char* e = std::getenv("RUSTORCH_QF_CTAS_PER_SM");
    return e ? std::max(1, std::atoi(e)) : 8;
  }();
  const int resident = sm_count(device) * std::max(std::min(per_sm, cap), 1);
  const dim3 grid(std::min((outs + per_cta - 1) / per_cta, resident)), block(QF_WARPS * 32);
  launch_pdl(kern, grid, block, smem, s, a.qs, reinterpret_cast<const __half*>(a.scales), reinterpret_cast<const __half*>(a.x),
             a.ldx, reinterpret_cast<const __half*>(a.norm_w), a.eps, reinterpret_cast<__half*>(a.y), a.ldy,
             reinterpret_cast<const __half*>(a.residual), a.ldr, a.N, a.K, reinterpret_cast<const uint8_t*>(a.prefetch0),
             a.prefetch0_bytes, reinterpret_cast<const uint8_t*>(a.prefetch1), a.prefetch1_bytes, rope);
  RT_LAUNCH_CHECK();
}

bool q_gemv_fused_supported(int M, int N, int K, bool swiglu) {
  return M >= 1 && M <= 4 && K % 64 == 0 && size_t(M) * (K + (K / 32) * 8) <= 100 * 1024 && (!swiglu || N % 2 == 0);
}

void q_gemv_fused(const QGemvFusedArgs& a, cudaStream_t stream) {
  RT_CHECK(q_gemv_fused_supported(a.M, a.N, a.K, a.swiglu), "q_gemv_fused: 1..4 rows, K a multiple of 64 that fits shared memory");
  RT_CHECK(a.ldx % 4 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 7) == 0 && (reinterpret_cast<uintptr_t>(a.qs) & 15) == 0,
           "q_gemv_fused: x rows must be 8-byte and qs 16-byte aligned");
  RT_CHECK(a.norm_w == nullptr || (reinterpret_cast<uintptr_t>(a.norm_w) & 7) == 0, "q_gemv_fused: norm weight must be 8-byte aligned");
  RT_CHECK(!(a.swiglu && a.residual), "q_gemv_fused: the SwiGLU epilogue takes no residual");
  RT_CHECK((long long)a.N * (a.K / 32) < (1LL << 31), "q_gemv_fused: weight matrix too large for 32-bit block offsets");
  RT_CHECK((reinterpret_cast<uintptr_t>(a.prefetch0) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.prefetch1) & 15) == 0,
           "q_gemv_fused: prefetch ranges must be 16-byte aligned");
  if (a.rope_pos != nullptr) {
    RT_CHECK(!a.swiglu && a.residual == nullptr, "q_gemv_fused: the rotary epilogue excludes SwiGLU and the residual");
    RT_CHECK(a.rope_D % 2 == 0 && a.rope_D > 0 && a.N == (a.rope_H + 2 * a.rope_Hkv) * a.rope_D && a.N % 4 == 0,
             "q_gemv_fused: rotary epilogue needs N = (H + 2 Hkv) D rows, D even");
    RT_CHECK(a.rope_seq != nullptr && a.cache_k != nullptr && a.cache_v != nullptr && a.rope_T_max > 0 && a.rope_n_seq > 0,
             "q_gemv_fused: rotary epilogue needs positions, sequence numbers and both caches");
  }
  if (a.N == 0) return;
#define RT_QF(Q8, MM)                                           \
  if (a.swiglu) launch_fused<Q8, MM, 1>(a, stream);             \
  else if (a.rope_pos != nullptr) launch_fused<Q8, MM, 2>(a, stream); \
  else launch_fused<Q8, MM, 0>(a, stream);
#define RT_QF_M(Q8)                   \
  switch (a.M) {                      \
    case 1: RT_QF(Q8, 1) break;       \
    case 2: RT_QF(Q8, 2) break;       \
    case 3: RT_QF(Q8, 3) break;       \
    default: RT_QF(Q8, 4) break;      \
  }
  if (a.q8) {
    RT_QF_M(true)
  } else {
    RT_QF_M(false)
  }
#undef RT_QF_M
#undef RT_QF
}

}  // namespace rt
