// Flash-attention backward on tcgen05 (sm_100a).  Two kernels, both recomputing the score
// tile from Q/K and the saved log-sum-exp, so nothing T x T is ever stored:
//
//   attn_bwd_dkdv : one CTA per (key tile j, kv head, batch); loops over the query tiles that can
//                   see it (and over the query heads of the GQA group), accumulating in TMEM
//                     dV += P^T dO         dK += dS^T Q
//   attn_bwd_dq   : one CTA per (query tile i, head, batch); loops over key tiles, accumulating
//                     dQ += dS K
//   with P = exp2(S*scale*log2e - lse*log2e), dS = P * (dP - delta), dP = dO V^T,
//   delta = rowsum(O * dO) from a small pre-pass kernel.
//
// Thread/TMEM mapping: score row r is owned by lane r % 32 of the two warps with warp % 4 == r / 32; the one with
// warp < 4 handles columns 0..63 of the tile, the other columns 64..127 (the softmax phase is latency bound, so
// eight warps finish it in about half the time of four).  P and
// dS go to the swizzled staging tiles, which serve as MN-major A operands (transposed use)
// in dkdv and as a K-major A operand in dq.  The reference has no attention backward at all
// (its head reshapes detach the graph, src/nn/attention.rs:255-289).
#include <cstdlib>

#include "../api.h"
#include "../common/launch.h"
#include "attn_common.cuh"

namespace rt {

void attn_bwd_fused_d64(const AttnArgs& a, cudaStream_t stream);  // flash_bwd_fused.cu

struct AttnBwdParams {
  int B, H, Hkv, Tq, Tk;
  int causal;
  float scale, scale_log2;
  const float* lse;    // [B][H][Tq]
  const float* delta;  // [B][H][Tq]
  __nv_bfloat16 *dq, *dk, *dv;
  long long dq_sb, dq_st, dq_sh, dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh;
  int* status;
};

// 8 softmax warps (two column halves x four TMEM lane quarters) + 1 control warp (TMA + MMA issue, TMEM owner).
constexpr int ATT_BWD_THREADS = 288;
constexpr int ATT_BWD_CTRL_WARP = 8;

// --------------------------------------------------------------------- delta pre-pass
// delta[b][h][t] = sum_d o[b][t][h][d] * do[b][t][h][d].  D/8 lanes per row, one 16-byte load
// per lane per tensor, so a warp covers 4 rows (D = 64) or 2 rows (D = 128).
template <int D>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                  int B, int H, int T, long long sb, long long st, long long sh) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  constexpr int LPR = D / 8;  // lanes per row
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gt / LPR;
  const int sub = int(gt % LPR);
  const long long rows = (long long)B * H * T;
  float acc = 0.f;
  if (row < rows) {
    const int t = int(row % T);
    const int h = int((row / T) % H);
    const int b = int(row / ((long long)T * H));
    const long long off = b * sb + t * st + h * sh + sub * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o + off);
    const uint4 c = *reinterpret_cast<const uint4*>(d_o + off);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(ha[e]), y = __bfloat1622float2(hc[e]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (row < rows && sub == 0) delta[row] = acc;
}

// ------------------------------------------------------------------------ dK / dV
template <int D>
struct DkDvSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int QSTAGES = (D == 64) ? 2 : 1;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;                    // QSTAGES tiles
  static constexpr int OFF_DO = OFF_Q + QSTAGES * TILE;     // QSTAGES tiles
  static constexpr int OFF_P = OFF_DO + QSTAGES * TILE;     // 32 KB
  static constexpr int OFF_DS = OFF_P + 2 * ATT_HALF_BYTES; // 32 KB
  static constexpr int OFF_BAR = OFF_DS + 2 * ATT_HALF_BYTES;
  // kv_full, qdo_full[2], qdo_empty[2], sdp_full, pds_full, pds_empty, done
  static constexpr int TOTAL = OFF_BAR + 9 * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q,
                     const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v,
                     const __grid_constant__ CUtensorMap tmap_do, const AttnBwdParams p) {
  using S = DkDvSmem<D>;
  constexpr int QS = S::QSTAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* pds_empty = bars + 7;
  uint64_t* done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * ATT_BN;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int group = p.H / p.Hkv;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 256);
    mbar_init(pds_empty, 1);
    mbar_init(done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == ATT_BWD_CTRL_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_dP = tmem_base + 128;
  const uint32_t tmem_dV = tmem_base + 256;
  const uint32_t tmem_dK = tmem_base + 256 + D;

  const int off = p.Tk - p.Tq;
  const int n_q = (p.Tq + ATT_BM - 1) / ATT_BM;
  int i_start = 0;
  if (p.causal) i_start = max(0, (k0 - off)) / ATT_BM;  // first query tile that sees column k0
  const int per_head = max(0, n_q - i_start);
  const int n_it = per_head * group;

  if (warp == ATT_BWD_CTRL_WARP) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_T = make_idesc_f16(128, D, true, true, true);  // P^T dO, dS^T Q
      bool ok = true;
      mbar_arrive_expect_tx(kv_full, 2 * S::TILE);
      load_tile<D>(smem + S::OFF_K, &tmap_k, kv_full, k0, hk, b);
      load_tile<D>(smem + S::OFF_V, &tmap_v, kv_full, k0, hk, b);
      // first Q/dO tile
      {
        const int h = hk * group;
        mbar_arrive_expect_tx(&qdo_full[0], 2 * S::TILE);
        load_tile<D>(smem + S::OFF_Q, &tmap_q, &qdo_full[0], i_start * ATT_BM, h, b);
        load_tile<D>(smem + S::OFF_DO, &tmap_do, &qdo_full[0], i_start * ATT_BM, h, b);
      }
      ok = mbar_wait(kv_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      const uint32_t aK = smem_u32(smem + S::OFF_K);
      const uint32_t aV = smem_u32(smem + S::OFF_V);
      const uint32_t aP = smem_u32(smem + S::OFF_P);
      const uint32_t aDS = smem_u32(smem + S::OFF_DS);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % QS;
        if (QS == 2 && it + 1 < n_it) {
          const int n = it + 1;
          const int s2 = n % QS;
          if (!mbar_wait(&qdo_empty[s2], ((n / QS) & 1) ^ 1, ctl, p.status,
                         RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const int h = hk * group + n / per_head;
          const int qi0 = (i_start + n % per_head) * ATT_BM;
          mbar_arrive_expect_tx(&qdo_full[s2], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_Q + s2 * S::TILE, &tmap_q, &qdo_full[s2], qi0, h, b);
          load_tile<D>(smem + S::OFF_DO + s2 * S::TILE, &tmap_do, &qdo_full[s2], qi0, h, b);
        }
        if (!mbar_wait(&qdo_full[s], (it / QS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t aQ = smem_u32(smem + S::OFF_Q + s * S::TILE);
        const uint32_t aDO = smem_u32(smem + S::OFF_DO + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S,
                      kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_dP, tile_desc_kmajor<D>(aDO, kk), tile_desc_kmajor<D>(aV, kk), idesc_S,
                      kk > 0 ? 1u : 0u);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, it & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < ATT_BM / 16; ++kk)
          umma_f16_ss(tmem_dV, stage_desc_mnmajor(aP, kk), tile_desc_mnmajor<D>(aDO, kk), idesc_T,
                      (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < ATT_BM / 16; ++kk)
          umma_f16_ss(tmem_dK, stage_desc_mnmajor(aDS, kk), tile_desc_mnmajor<D>(aQ, kk), idesc_T,
                      (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&qdo_empty[s]);
        umma_commit(pds_empty);
        if (QS == 1 && it + 1 < n_it) {
          // single-stage ring: reload after the MMAs that read this stage retire
          const int n = it + 1;
          if (!mbar_wait(&qdo_empty[0], (it & 1), ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const int h = hk * group + n / per_head;
          const int qi0 = (i_start + n % per_head) * ATT_BM;
          mbar_arrive_expect_tx(&qdo_full[0], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_Q, &tmap_q, &qdo_full[0], qi0, h, b);
          load_tile<D>(smem + S::OFF_DO, &tmap_do, &qdo_full[0], qi0, h, b);
        }
      }
      if (ok) umma_commit(done);
    }
  } else {
    // warps 0..3 take score columns 0..63, warps 4..7 columns 64..127 of the same 128 rows
    const int quarter = warp & 3, chalf = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint8_t* sP = smem + S::OFF_P;
    uint8_t* sDS = smem + S::OFF_DS;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * group + it / per_head;
      const int qi = (i_start + it % per_head) * ATT_BM + row;
      const bool row_ok = qi < p.Tq;
      const long long sidx = ((long long)b * p.H + h) * p.Tq + qi;
      const float lse2 = row_ok ? p.lse[sidx] * 1.4426950408889634f : 0.f;
      const float dl = row_ok ? p.delta[sidx] : 0.f;
      const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);
      if (!mbar_wait(sdp_full, it & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      if (it > 0 && !mbar_wait(pds_empty, (it - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // all four TMEM loads of this thread's 64 columns are issued before the single wait
      uint32_t rs[2][32], rp[2][32];
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        tmem_ld_32x32b_x32(tmem_S + lane_sel + (chalf * 2 + u) * 32, rs[u]);
        tmem_ld_32x32b_x32(tmem_dP + lane_sel + (chalf * 2 + u) * 32, rp[u]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
        float pv[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool vis = row_ok && (k0 + c * 32 + i <= limit);
          const float e = vis ? ex2_approx(__uint_as_float(rs[u][i]) * p.scale_log2 - lse2) : 0.f;
          pv[i] = e;
          ds[i] = e * (__uint_as_float(rp[u][i]) - dl);
        }
        stage_row_chunk_bf16(sP, row, c * 32, pv);
        stage_row_chunk_bf16(sDS, row, c * 32, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
    }
    // final: thread t owns key row k0 + t of dK / dV
    if (n_it > 0 && ok) ok = mbar_wait(done, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
    tc_fence_after();
    const int kr = k0 + row;
#pragma unroll 1
    for (int which = chalf; which < chalf + 1; ++which) {  // column half 0 writes dV, half 1 writes dK
      const uint32_t src = which == 0 ? tmem_dV : tmem_dK;
      const float mul = which == 0 ? 1.f : p.scale;
      __nv_bfloat16* dst =
          which == 0
              ? p.dv + (long long)b * p.dv_sb + (long long)kr * p.dv_st + (long long)hk * p.dv_sh
              : p.dk + (long long)b * p.dk_sb + (long long)kr * p.dk_st + (long long)hk * p.dk_sh;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (n_it > 0 && ok) {
          __syncwarp();
          tmem_ld_32x32b_x32(src + lane_sel + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (kr < p.Tk) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul);
            w.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul);
            w.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul);
            w.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul);
            reinterpret_cast<uint4*>(dst + c * 32)[q] = w;
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_BWD_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- dQ
template <int D>
struct DqSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int KSTAGES = (D == 64) ? 2 : 1;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;
  static constexpr int OFF_V = OFF_K + KSTAGES * TILE;
  static constexpr int OFF_DS = OFF_V + KSTAGES * TILE;
  static constexpr int OFF_BAR = OFF_DS + 2 * ATT_HALF_BYTES;
  // qdo_full, kv_full[2], kv_empty[2], sdp_full, ds_full, ds_empty, done
  static constexpr int TOTAL = OFF_BAR + 9 * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v,
                   const __grid_constant__ CUtensorMap tmap_do, const AttnBwdParams p) {
  using S = DqSmem<D>;
  constexpr int KS = S::KSTAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;
  uint64_t* ds_full = bars + 6;
  uint64_t* ds_empty = bars + 7;
  uint64_t* done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * ATT_BM;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(ds_empty, 1);
    mbar_init(done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == ATT_BWD_CTRL_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_dP = tmem_base + 128;
  const uint32_t tmem_dQ = tmem_base + 256;

  const int off = p.Tk - p.Tq;
  int n_kv = (p.Tk + ATT_BN - 1) / ATT_BN;
  if (p.causal) {
    const int last_col = min(p.Tk - 1, q0 + ATT_BM - 1 + off);
    n_kv = last_col < 0 ? 0 : min(n_kv, last_col / ATT_BN + 1);
  }

  if (warp == ATT_BWD_CTRL_WARP) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_Q = make_idesc_f16(128, D, false, true, true);  // dS @ K
      bool ok = true;
      mbar_arrive_expect_tx(qdo_full, 2 * S::TILE);
      load_tile<D>(smem + S::OFF_Q, &tmap_q, qdo_full, q0, h, b);
      load_tile<D>(smem + S::OFF_DO, &tmap_do, qdo_full, q0, h, b);
      mbar_arrive_expect_tx(&kv_full[0], 2 * S::TILE);
      load_tile<D>(smem + S::OFF_K, &tmap_k, &kv_full[0], 0, hk, b);
      load_tile<D>(smem + S::OFF_V, &tmap_v, &kv_full[0], 0, hk, b);
      ok = mbar_wait(qdo_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      const uint32_t aQ = smem_u32(smem + S::OFF_Q);
      const uint32_t aDO = smem_u32(smem + S::OFF_DO);
      const uint32_t aDS = smem_u32(smem + S::OFF_DS);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KS;
        if (KS == 2 && j + 1 < n_kv) {
          const int n = j + 1;
          const int s2 = n % KS;
          if (!mbar_wait(&kv_empty[s2], ((n / KS) & 1) ^ 1, ctl, p.status,
                         RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[s2], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_K + s2 * S::TILE, &tmap_k, &kv_full[s2], n * ATT_BN, hk, b);
          load_tile<D>(smem + S::OFF_V + s2 * S::TILE, &tmap_v, &kv_full[s2], n * ATT_BN, hk, b);
        }
        if (!mbar_wait(&kv_full[s], (j / KS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t aK = smem_u32(smem + S::OFF_K + s * S::TILE);
        const uint32_t aV = smem_u32(smem + S::OFF_V + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S,
                      kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_dP, tile_desc_kmajor<D>(aDO, kk), tile_desc_kmajor<D>(aV, kk), idesc_S,
                      kk > 0 ? 1u : 0u);
        umma_commit(sdp_full);
        if (!mbar_wait(ds_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          umma_f16_ss(tmem_dQ, stage_desc_kmajor(aDS, kk), tile_desc_mnmajor<D>(aK, kk), idesc_Q,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(ds_empty);
        if (KS == 1 && j + 1 < n_kv) {
          const int n = j + 1;
          if (!mbar_wait(&kv_empty[0], (j & 1), ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[0], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_K, &tmap_k, &kv_full[0], n * ATT_BN, hk, b);
          load_tile<D>(smem + S::OFF_V, &tmap_v, &kv_full[0], n * ATT_BN, hk, b);
        }
      }
      if (ok) umma_commit(done);
    }
  } else {
    const int quarter = warp & 3, chalf = warp >> 2;
    const int row = quarter * 32 + lane;
    const int qi = q0 + row;
    const bool row_ok = qi < p.Tq;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint8_t* sDS = smem + S::OFF_DS;
    const long long sidx = ((long long)b * p.H + h) * p.Tq + qi;
    const float lse2 = row_ok ? p.lse[sidx] * 1.4426950408889634f : 0.f;
    const float dl = row_ok ? p.delta[sidx] : 0.f;
    const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(sdp_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      if (j > 0 && !mbar_wait(ds_empty, (j - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t rs[2][32], rp[2][32];
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        tmem_ld_32x32b_x32(tmem_S + lane_sel + (chalf * 2 + u) * 32, rs[u]);
        tmem_ld_32x32b_x32(tmem_dP + lane_sel + (chalf * 2 + u) * 32, rp[u]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
        float ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool vis = row_ok && (j * ATT_BN + c * 32 + i <= limit);
          const float e = vis ? ex2_approx(__uint_as_float(rs[u][i]) * p.scale_log2 - lse2) : 0.f;
          ds[i] = e * (__uint_as_float(rp[u][i]) - dl);
        }
        stage_row_chunk_bf16(sDS, row, c * 32, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_full);
    }
    if (n_kv > 0 && ok) ok = mbar_wait(done, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
    tc_fence_after();
    __nv_bfloat16* dst =
        p.dq + (long long)b * p.dq_sb + (long long)qi * p.dq_st + (long long)h * p.dq_sh;
#pragma unroll 1
    for (int c = chalf * (D / 64); c < (chalf + 1) * (D / 64); ++c) {
      uint32_t r[32];
      if (n_kv > 0 && ok) {
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_dQ + lane_sel + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale);
          w.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale);
          w.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale);
          w.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale);
          reinterpret_cast<uint4*>(dst + c * 32)[q] = w;
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_BWD_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------ dK / dV, pipelined (D = 64)
// The kernel above runs MMA(S, dP) -> softmax -> MMA(dV, dK) as a serial chain per (kv block, q block) pair.  With
// 64-wide heads tensor memory has room for a second S accumulator (2 x 128 + 128 + 64 + 64 = 512 columns), so here
// the control thread issues S of pair i+1 before it waits for the softmax warps of pair i, and dP of pair i+1
// directly after that wait, ahead of dV / dK of pair i: the exponentials of pair i+1 then run under the dV / dK
// MMAs of pair i.  Q / dO tiles sit in a three-stage ring so that the loads of pair i+2 never wait on those MMAs.
struct DkDvPipeSmem {
  static constexpr int TILE = 128 * 64 * 2;
  static constexpr int QSTAGES = 3;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;
  static constexpr int OFF_DO = OFF_Q + QSTAGES * TILE;
  static constexpr int OFF_P = OFF_DO + QSTAGES * TILE;
  static constexpr int OFF_DS = OFF_P + 2 * ATT_HALF_BYTES;
  static constexpr int OFF_BAR = OFF_DS + 2 * ATT_HALF_BYTES;
  // kv_full, qdo_full[3], qdo_empty[3], s_full[2], dp_full, pds_full, pds_empty, done
  static constexpr int TOTAL = OFF_BAR + 13 * 8 + 16;
};

__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attn_bwd_dkdv_pipe_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                          const AttnBwdParams p) {
  constexpr int D = 64;
  using S = DkDvPipeSmem;
  constexpr int QS = S::QSTAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 4;
  uint64_t* s_full = bars + 7;
  uint64_t* dp_full = bars + 9;
  uint64_t* pds_full = bars + 10;
  uint64_t* pds_empty = bars + 11;
  uint64_t* done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * ATT_BN;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int group = p.H / p.Hkv;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, 256);
    mbar_init(pds_empty, 1);
    mbar_init(done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == ATT_BWD_CTRL_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;  // S of pair i lives at tmem_S0 + (i & 1) * 128
  const uint32_t tmem_dP = tmem_base + 256;
  const uint32_t tmem_dV = tmem_base + 384;
  const uint32_t tmem_dK = tmem_base + 448;

  const int off = p.Tk - p.Tq;
  const int n_q = (p.Tq + ATT_BM - 1) / ATT_BM;
  int i_start = 0;
  if (p.causal) i_start = max(0, (k0 - off)) / ATT_BM;
  const int per_head = max(0, n_q - i_start);
  const int n_it = per_head * group;

  if (warp == ATT_BWD_CTRL_WARP) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_T = make_idesc_f16(128, D, true, true, true);  // P^T dO, dS^T Q
      bool ok = true;
      const uint32_t aK = smem_u32(smem + S::OFF_K);
      const uint32_t aV = smem_u32(smem + S::OFF_V);
      const uint32_t aP = smem_u32(smem + S::OFF_P);
      const uint32_t aDS = smem_u32(smem + S::OFF_DS);
      auto load_q = [&](int n) {  // Q / dO tiles of pair n into ring stage n % QS (after the MMAs of pair n - QS retired)
        const int st = n % QS;
        if (!mbar_wait(&qdo_empty[st], ((n / QS) & 1) ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
        const int h = hk * group + n / per_head;
        const int qi0 = (i_start + n % per_head) * ATT_BM;
        mbar_arrive_expect_tx(&qdo_full[st], 2 * S::TILE);
        load_tile<D>(smem + S::OFF_Q + st * S::TILE, &tmap_q, &qdo_full[st], qi0, h, b);
        load_tile<D>(smem + S::OFF_DO + st * S::TILE, &tmap_do, &qdo_full[st], qi0, h, b);
        return true;
      };
      auto issue_S = [&](int n) {
        const uint32_t aQ = smem_u32(smem + S::OFF_Q + (n % QS) * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S0 + (n & 1) * 128, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[n & 1]);
      };
      auto issue_dP = [&](int n) {
        const uint32_t aDO = smem_u32(smem + S::OFF_DO + (n % QS) * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_dP, tile_desc_kmajor<D>(aDO, kk), tile_desc_kmajor<D>(aV, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(dp_full);
      };
      mbar_arrive_expect_tx(kv_full, 2 * S::TILE);
      load_tile<D>(smem + S::OFF_K, &tmap_k, kv_full, k0, hk, b);
      load_tile<D>(smem + S::OFF_V, &tmap_v, kv_full, k0, hk, b);
      ok = load_q(0);
      if (ok && n_it > 1) ok = load_q(1);
      ok = ok && mbar_wait(kv_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      ok = ok && mbar_wait(&qdo_full[0], 0, ctl, p.status, RT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_S(0);
        issue_dP(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          const int n = it + 1;
          if (!mbar_wait(&qdo_full[n % QS], (n / QS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_S(n);  // its buffer was last read by the softmax warps of pair n - 2, which finished before pds_full(n - 2)
        }
        if (it + 2 < n_it && !load_q(it + 2)) {
          ok = false;
          break;
        }
        if (!mbar_wait(pds_full, it & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (it + 1 < n_it) issue_dP(it + 1);  // ahead of dV / dK: the softmax warps of pair it + 1 need it first
        const int s = it % QS;
        const uint32_t aQ = smem_u32(smem + S::OFF_Q + s * S::TILE);
        const uint32_t aDO = smem_u32(smem + S::OFF_DO + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < ATT_BM / 16; ++kk)
          umma_f16_ss(tmem_dV, stage_desc_mnmajor(aP, kk), tile_desc_mnmajor<D>(aDO, kk), idesc_T, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < ATT_BM / 16; ++kk)
          umma_f16_ss(tmem_dK, stage_desc_mnmajor(aDS, kk), tile_desc_mnmajor<D>(aQ, kk), idesc_T, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&qdo_empty[s]);
        umma_commit(pds_empty);
      }
      if (ok) umma_commit(done);
    }
  } else {
    // warps 0..3 take score columns 0..63, warps 4..7 columns 64..127 of the same 128 rows
    const int quarter = warp & 3, chalf = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint8_t* sP = smem + S::OFF_P;
    uint8_t* sDS = smem + S::OFF_DS;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * group + it / per_head;
      const int qi = (i_start + it % per_head) * ATT_BM + row;
      const bool row_ok = qi < p.Tq;
      const long long sidx = ((long long)b * p.H + h) * p.Tq + qi;
      const float lse2 = row_ok ? p.lse[sidx] * 1.4426950408889634f : 0.f;
      const float dl = row_ok ? p.delta[sidx] : 0.f;
      const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);
      if (!mbar_wait(&s_full[it & 1], (it >> 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t rs[2][32], rp[2][32];
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_S0 + (it & 1) * 128 + lane_sel + (chalf * 2 + u) * 32, rs[u]);
      tmem_ld_wait();
      // probabilities first (they only need S); rs is reused for them
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool vis = row_ok && (k0 + c * 32 + i <= limit);
          rs[u][i] = __float_as_uint(vis ? ex2_approx(__uint_as_float(rs[u][i]) * p.scale_log2 - lse2) : 0.f);
        }
      }
      if (!mbar_wait(dp_full, it & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_dP + lane_sel + (chalf * 2 + u) * 32, rp[u]);
      tmem_ld_wait();
      if (it > 0 && !mbar_wait(pds_empty, (it - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
        float pv[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pv[i] = __uint_as_float(rs[u][i]);
          ds[i] = pv[i] * (__uint_as_float(rp[u][i]) - dl);
        }
        stage_row_chunk_bf16(sP, row, c * 32, pv);
        stage_row_chunk_bf16(sDS, row, c * 32, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
    }
    // final: thread t owns key row k0 + t of dK / dV
    if (n_it > 0 && ok) ok = mbar_wait(done, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
    tc_fence_after();
    const int kr = k0 + row;
    const uint32_t src = chalf == 0 ? tmem_dV : tmem_dK;  // column half 0 writes dV, half 1 writes dK
    const float mul = chalf == 0 ? 1.f : p.scale;
    __nv_bfloat16* dst = chalf == 0 ? p.dv + (long long)b * p.dv_sb + (long long)kr * p.dv_st + (long long)hk * p.dv_sh
                                    : p.dk + (long long)b * p.dk_sb + (long long)kr * p.dk_st + (long long)hk * p.dk_sh;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (n_it > 0 && ok) {
        __syncwarp();
        tmem_ld_32x32b_x32(src + lane_sel + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (kr < p.Tk) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul);
          w.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul);
          w.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul);
          w.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul);
          reinterpret_cast<uint4*>(dst + c * 32)[q] = w;
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_BWD_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------ dQ, pipelined (D = 64)
// Same scheme as the pipelined dK / dV kernel: S of kv block j+1 goes to the second S accumulator before the control
// thread waits for the softmax warps of block j, dP of block j+1 is issued ahead of dQ += dS K of block j, and the
// K / V tiles sit in a three-stage ring.  Tensor memory: 2 x 128 (S) + 128 (dP) + 64 (dQ) = 448 columns.
struct DqPipeSmem {
  static constexpr int TILE = 128 * 64 * 2;
  static constexpr int KSTAGES = 3;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;
  static constexpr int OFF_V = OFF_K + KSTAGES * TILE;
  static constexpr int OFF_DS = OFF_V + KSTAGES * TILE;
  static constexpr int OFF_BAR = OFF_DS + 2 * ATT_HALF_BYTES;
  // qdo_full, kv_full[3], kv_empty[3], s_full[2], dp_full, ds_full, ds_empty, done
  static constexpr int TOTAL = OFF_BAR + 13 * 8 + 16;
};

__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attn_bwd_dq_pipe_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                        const AttnBwdParams p) {
  constexpr int D = 64;
  using S = DqPipeSmem;
  constexpr int KS = S::KSTAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 4;
  uint64_t* s_full = bars + 7;
  uint64_t* dp_full = bars + 9;
  uint64_t* ds_full = bars + 10;
  uint64_t* ds_empty = bars + 11;
  uint64_t* done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * ATT_BM;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(ds_empty, 1);
    mbar_init(done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == ATT_BWD_CTRL_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;  // S of block j at tmem_S0 + (j & 1) * 128
  const uint32_t tmem_dP = tmem_base + 256;
  const uint32_t tmem_dQ = tmem_base + 384;

  const int off = p.Tk - p.Tq;
  int n_kv = (p.Tk + ATT_BN - 1) / ATT_BN;
  if (p.causal) {
    const int last_col = min(p.Tk - 1, q0 + ATT_BM - 1 + off);
    n_kv = last_col < 0 ? 0 : min(n_kv, last_col / ATT_BN + 1);
  }

  if (warp == ATT_BWD_CTRL_WARP) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_Q = make_idesc_f16(128, D, false, true, true);  // dS @ K
      bool ok = true;
      const uint32_t aQ = smem_u32(smem + S::OFF_Q);
      const uint32_t aDO = smem_u32(smem + S::OFF_DO);
      const uint32_t aDS = smem_u32(smem + S::OFF_DS);
      auto load_kv = [&](int n) {
        const int st = n % KS;
        if (!mbar_wait(&kv_empty[st], ((n / KS) & 1) ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
        mbar_arrive_expect_tx(&kv_full[st], 2 * S::TILE);
        load_tile<D>(smem + S::OFF_K + st * S::TILE, &tmap_k, &kv_full[st], n * ATT_BN, hk, b);
        load_tile<D>(smem + S::OFF_V + st * S::TILE, &tmap_v, &kv_full[st], n * ATT_BN, hk, b);
        return true;
      };
      auto issue_S = [&](int n) {
        const uint32_t aK = smem_u32(smem + S::OFF_K + (n % KS) * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S0 + (n & 1) * 128, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[n & 1]);
      };
      auto issue_dP = [&](int n) {
        const uint32_t aV = smem_u32(smem + S::OFF_V + (n % KS) * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_dP, tile_desc_kmajor<D>(aDO, kk), tile_desc_kmajor<D>(aV, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(dp_full);
      };
      mbar_arrive_expect_tx(qdo_full, 2 * S::TILE);
      load_tile<D>(smem + S::OFF_Q, &tmap_q, qdo_full, q0, h, b);
      load_tile<D>(smem + S::OFF_DO, &tmap_do, qdo_full, q0, h, b);
      ok = load_kv(0);
      if (ok && n_kv > 1) ok = load_kv(1);
      ok = ok && mbar_wait(qdo_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      ok = ok && mbar_wait(&kv_full[0], 0, ctl, p.status, RT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_S(0);
        issue_dP(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int n = j + 1;
          if (!mbar_wait(&kv_full[n % KS], (n / KS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_S(n);
        }
        if (j + 2 < n_kv && !load_kv(j + 2)) {
          ok = false;
          break;
        }
        if (!mbar_wait(ds_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (j + 1 < n_kv) issue_dP(j + 1);
        const int s = j % KS;
        const uint32_t aK = smem_u32(smem + S::OFF_K + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          umma_f16_ss(tmem_dQ, stage_desc_kmajor(aDS, kk), tile_desc_mnmajor<D>(aK, kk), idesc_Q, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(ds_empty);
      }
      if (ok) umma_commit(done);
    }
  } else {
    const int quarter = warp & 3, chalf = warp >> 2;
    const int row = quarter * 32 + lane;
    const int qi = q0 + row;
    const bool row_ok = qi < p.Tq;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint8_t* sDS = smem + S::OFF_DS;
    const long long sidx = ((long long)b * p.H + h) * p.Tq + qi;
    const float lse2 = row_ok ? p.lse[sidx] * 1.4426950408889634f : 0.f;
    const float dl = row_ok ? p.delta[sidx] : 0.f;
    const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t rs[2][32], rp[2][32];
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_S0 + (j & 1) * 128 + lane_sel + (chalf * 2 + u) * 32, rs[u]);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool vis = row_ok && (j * ATT_BN + c * 32 + i <= limit);
          rs[u][i] = __float_as_uint(vis ? ex2_approx(__uint_as_float(rs[u][i]) * p.scale_log2 - lse2) : 0.f);
        }
      }
      if (!mbar_wait(dp_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_dP + lane_sel + (chalf * 2 + u) * 32, rp[u]);
      tmem_ld_wait();
      if (j > 0 && !mbar_wait(ds_empty, (j - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = chalf * 2 + u;
        float ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) ds[i] = __uint_as_float(rs[u][i]) * (__uint_as_float(rp[u][i]) - dl);
        stage_row_chunk_bf16(sDS, row, c * 32, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_full);
    }
    if (n_kv > 0 && ok) ok = mbar_wait(done, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
    tc_fence_after();
    __nv_bfloat16* dst = p.dq + (long long)b * p.dq_sb + (long long)qi * p.dq_st + (long long)h * p.dq_sh;
    {
      const int c = chalf;  // 32 of the 64 columns per column half
      uint32_t r[32];
      if (n_kv > 0 && ok) {
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_dQ + lane_sel + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale);
          w.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale);
          w.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale);
          w.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale);
          reinterpret_cast<uint4*>(dst + c * 32)[q] = w;
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ATT_BWD_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static void launch_bwd(const AttnArgs& a, cudaStream_t stream) {
  const int device = current_device();
  auto k1 = attn_bwd_dkdv_kernel<D>;
  auto k2 = attn_bwd_dq_kernel<D>;
  static bool configured[64] = {false};
  if (!configured[device]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       DkDvSmem<D>::TOTAL));
    RT_CUDA_CHECK(
        cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<D>::TOTAL));
    configured[device] = true;
  }
  {
    const long long threads = (long long)a.B * a.H * a.Tq * (D / 8);
    attn_delta_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(a.o), reinterpret_cast<const __nv_bfloat16*>(a.d_o),
        a.delta, a.B, a.H, a.Tq, a.o_sb, a.o_st, a.o_sh);
    RT_LAUNCH_CHECK();
  }
  // 64-wide heads with an accumulation buffer: one kernel computes dK, dV and dQ from a single S / dP per tile pair
  // (flash_bwd_fused.cu).  RUSTORCH_ATTN_BWD_FUSED=0 keeps the two-kernel path below.
  static const bool fused = [] {
    const char* e = std::getenv("RUSTORCH_ATTN_BWD_FUSED");
    return !(e && e[0] == '0');
  }();
  if (D == 64 && a.dq_acc != nullptr && fused) {
    attn_bwd_fused_d64(a, stream);
    return;
  }
  CUtensorMap tq = make_tmap_2byte_4d(a.q, D, a.Tq, a.H, a.B, a.q_st, a.q_sh, a.q_sb, 64, 128);
  CUtensorMap tk = make_tmap_2byte_4d(a.k, D, a.Tk, a.Hkv, a.B, a.k_st, a.k_sh, a.k_sb, 64, 128);
  CUtensorMap tv = make_tmap_2byte_4d(a.v, D, a.Tk, a.Hkv, a.B, a.v_st, a.v_sh, a.v_sb, 64, 128);
  CUtensorMap tdo = make_tmap_2byte_4d(a.d_o, D, a.Tq, a.H, a.B, a.o_st, a.o_sh, a.o_sb, 64, 128);
  AttnBwdParams p{};
  p.B = a.B;
  p.H = a.H;
  p.Hkv = a.Hkv;
  p.Tq = a.Tq;
  p.Tk = a.Tk;
  p.causal = a.causal;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.lse = a.lse;
  p.delta = a.delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(a.dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(a.dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(a.dv);
  p.dq_sb = a.dq_sb; p.dq_st = a.dq_st; p.dq_sh = a.dq_sh;
  p.dk_sb = a.dk_sb; p.dk_st = a.dk_st; p.dk_sh = a.dk_sh;
  p.dv_sb = a.dv_sb; p.dv_st = a.dv_st; p.dv_sh = a.dv_sh;
  p.status = status_word(device);
  {
    dim3 grid((a.Tk + ATT_BN - 1) / ATT_BN, a.Hkv, a.B);
    static const bool pipe = [] {  // RUSTORCH_ATTN_BWD_PIPE=0 falls back to the serial dK / dV kernel for 64-wide heads
      const char* e = std::getenv("RUSTORCH_ATTN_BWD_PIPE");
      return !(e && e[0] == '0');
    }();
    if (D == 64 && pipe) {
      static bool configured_pipe[64] = {false};
      if (!configured_pipe[device]) {
        RT_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkdv_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DkDvPipeSmem::TOTAL));
        configured_pipe[device] = true;
      }
      attn_bwd_dkdv_pipe_kernel<<<grid, ATT_BWD_THREADS, DkDvPipeSmem::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    } else {
      k1<<<grid, ATT_BWD_THREADS, DkDvSmem<D>::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    }
    RT_LAUNCH_CHECK();
  }
  {
    dim3 grid((a.Tq + ATT_BM - 1) / ATT_BM, a.H, a.B);
    static const bool pipe_dq = [] {  // RUSTORCH_ATTN_BWD_PIPE_DQ=0 falls back to the serial dQ kernel for 64-wide heads
      const char* e = std::getenv("RUSTORCH_ATTN_BWD_PIPE_DQ");
      return !(e && e[0] == '0');
    }();
    if (D == 64 && pipe_dq) {
      static bool configured_dq[64] = {false};
      if (!configured_dq[device]) {
        RT_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DqPipeSmem::TOTAL));
        configured_dq[device] = true;
      }
      attn_bwd_dq_pipe_kernel<<<grid, ATT_BWD_THREADS, DqPipeSmem::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    } else {
      k2<<<grid, ATT_BWD_THREADS, DqSmem<D>::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    }
    RT_LAUNCH_CHECK();
  }
}

void attn_bwd(const AttnArgs& a, cudaStream_t stream) {
  RT_CHECK(a.D == 64 || a.D == 128, "attention: head_dim must be 64 or 128");
  RT_CHECK(a.H % a.Hkv == 0, "attention: n_heads must be a multiple of n_kv_heads");
  if (a.B == 0 || a.Tq == 0) return;
  if (a.D == 64) launch_bwd<64>(a, stream);
  else launch_bwd<128>(a, stream);
}

}  // namespace rt
