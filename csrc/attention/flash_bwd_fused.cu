// Flash-attention backward for 64-wide heads in ONE persistent kernel (sm_100a): every (key tile, query tile) pair
// computes its scores and dP exactly once and feeds all three gradients,
//     S  = Q K^T                 dP = dO V^T                                  (tcgen05, fp32 in tensor memory)
//     P  = exp2(S scale log2e - lse log2e)      dS = P (dP - delta)           (256 softmax threads, 64 columns each)
//     dV += P^T dO               dK += dS^T Q                                 (accumulated in tensor memory per key tile)
//     dQ_partial = dS K          -> TMA reduce-add of fp32 tiles into a dQ accumulation buffer (scale folded in)
// instead of one kernel that recomputes S / dP for dK, dV and a second one that recomputes them again for dQ.
//
// A CTA (one per SM) walks a list of work items; an item is one key tile of one (batch, kv head) and all the query
// tiles (of all query heads of the GQA group) that can see it.  Items are dealt longest first to the least loaded
// CTA on the host.  Tensor memory (512 columns): S ping | S pong | dP | dV | dK.  The control thread issues S of
// pair g+1 while the softmax warps still work on pair g, and dP of pair g+1 ahead of the dV / dK MMAs of pair g;
// dQ_partial of pair g is written over the S buffer of pair g (its scores are in registers by then) and drained by
// the softmax warps during pair g+1.  Q / dO tiles stream through a three-stage TMA ring that runs across items.
// A small kernel afterwards turns the fp32 dQ accumulation into bf16.  The reference has no attention backward at
// all (its head reshapes detach the graph, src/nn/attention.rs:255-289).
#include <algorithm>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <vector>

#include "../api.h"
#include "../common/launch.h"
#include "attn_common.cuh"

namespace rt {

struct AttnBwdFusedParams {
  int B, H, Hkv, Tq, Tk;
  int causal;
  float scale, scale_log2;
  const float* lse;    // [B][H][Tq]
  const float* delta;  // [B][H][Tq]
  float* dq_acc;       // fp32 [B][Tq][H][64], zero on entry
  __nv_bfloat16 *dk, *dv;
  long long dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh;
  const int* item_list;  // [gridDim.x][items_per_cta], -1 = none; item id = (batch * Hkv + kv head) * n_kv_tiles + key tile
  int items_per_cta;
  int n_kv_tiles;
  int* status;
};

constexpr int FB_THREADS = 288;  // 8 softmax warps (4 TMEM lane quarters x 2 column halves) + 1 control warp
constexpr int FB_CTRL_WARP = 8;
constexpr int FB_D = 64;

struct FusedBwdSmem {
  static constexpr int TILE = 128 * FB_D * 2;
  static constexpr int QSTAGES = 3;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;
  static constexpr int OFF_DO = OFF_Q + QSTAGES * TILE;
  static constexpr int OFF_P = OFF_DO + QSTAGES * TILE;
  static constexpr int OFF_DS = OFF_P + 2 * ATT_HALF_BYTES;
  static constexpr int OFF_DQ = OFF_DS + 2 * ATT_HALF_BYTES;   // 8 warps x (32 rows x 128 B) fp32 staging for the dQ reduce
  static constexpr int OFF_BAR = OFF_DQ + 8 * 4096;
  // kv_full, qdo_full[3], qdo_empty[3], s_full[2], dp_full, pds_full, pds_empty, dq_full, dq_drained, done, acc_free
  static constexpr int N_BARS = 16;
  static constexpr int TOTAL = OFF_BAR + N_BARS * 8 + 16;
  static_assert(TOTAL <= 232448, "attention backward: shared memory over the per-CTA limit");
};


// Geometry of one item.
struct FbItem {
  int b, hk, k0, i_start, per_head, n_it;
};
__device__ __forceinline__ bool fb_item(int k, const AttnBwdFusedParams& p, FbItem& it) {
  if (k >= p.items_per_cta) return false;
  const int id = __ldg(p.item_list + (long long)blockIdx.x * p.items_per_cta + k);
  if (id < 0) return false;
  const int jt = id % p.n_kv_tiles;
  const int bh = id / p.n_kv_tiles;
  it.hk = bh % p.Hkv;
  it.b = bh / p.Hkv;
  it.k0 = jt * ATT_BN;
  const int n_q = (p.Tq + ATT_BM - 1) / ATT_BM;
  it.i_start = p.causal ? max(0, it.k0 - (p.Tk - p.Tq)) / ATT_BM : 0;
  it.per_head = max(0, n_q - it.i_start);
  it.n_it = it.per_head * (p.H / p.Hkv);
  return true;
}

__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      const __grid_constant__ CUtensorMap tmap_dq, const AttnBwdFusedParams p) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  constexpr int D = FB_D;
  using S = FusedBwdSmem;
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
  uint64_t* dq_full = bars + 12;
  uint64_t* dq_drained = bars + 13;
  uint64_t* done = bars + 14;
  uint64_t* acc_free = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S::N_BARS);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
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
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 256);
    mbar_init(done, 1);
    mbar_init(acc_free, 256);
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_dq);
  }
  if (warp == FB_CTRL_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;  // S of pair g at tmem_S0 + (g & 1) * 128; dQ_partial of pair g reuses its first 64 columns
  const uint32_t tmem_dP = tmem_base + 256;
  const uint32_t tmem_dV = tmem_base + 384;
  const uint32_t tmem_dK = tmem_base + 448;
  const int off = p.Tk - p.Tq;

  if (warp == FB_CTRL_WARP) {
    // ================================================================== control thread: TMA + MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_T = make_idesc_f16(128, D, true, true, true);    // P^T dO, dS^T Q
      constexpr uint32_t idesc_Q = make_idesc_f16(128, D, false, true, true);   // dS K
      const uint32_t aK = smem_u32(smem + S::OFF_K);
      const uint32_t aV = smem_u32(smem + S::OFF_V);
      const uint32_t aP = smem_u32(smem + S::OFF_P);
      const uint32_t aDS = smem_u32(smem + S::OFF_DS);
      bool ok = true;
      uint32_t g_base = 0;   // pairs finished in earlier items (phase of the per-pair barriers, ring position)
      uint32_t items = 0;    // items with at least one pair so far
      for (int k = 0; ok; ++k) {
        FbItem itm;
        if (!fb_item(k, p, itm)) break;
        if (itm.n_it == 0) continue;  // the softmax warps write zeros for it
        const int n_it = itm.n_it;
        auto load_q = [&](int n) -> bool {  // Q / dO of pair n (item-local) into ring stage (g_base + n) % QS
          const uint32_t g = g_base + n;
          const int st = g % QS;
          if (!mbar_wait_idle(&qdo_empty[st], ((g / QS) & 1) ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
          const int h = itm.hk * group + n / itm.per_head;
          const int qi0 = (itm.i_start + n % itm.per_head) * ATT_BM;
          mbar_arrive_expect_tx(&qdo_full[st], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_Q + st * S::TILE, &tmap_q, &qdo_full[st], qi0, h, itm.b);
          load_tile<D>(smem + S::OFF_DO + st * S::TILE, &tmap_do, &qdo_full[st], qi0, h, itm.b);
          return true;
        };
        auto issue_S = [&](int n) {
          const uint32_t g = g_base + n;
          const uint32_t aQ = smem_u32(smem + S::OFF_Q + (g % QS) * S::TILE);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma_f16_ss(tmem_S0 + (g & 1) * 128, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S, kk > 0 ? 1u : 0u);
          umma_commit(&s_full[g & 1]);
        };
        auto issue_dP = [&](int n) {
          const uint32_t g = g_base + n;
          const uint32_t aDO = smem_u32(smem + S::OFF_DO + (g % QS) * S::TILE);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma_f16_ss(tmem_dP, tile_desc_kmajor<D>(aDO, kk), tile_desc_kmajor<D>(aV, kk), idesc_S, kk > 0 ? 1u : 0u);
          umma_commit(dp_full);
        };
        // The S buffer of pair g holds dQ_partial(g - 2) until the softmax warps have drained it.  For the first
        // pair of an item the wait is on pair g - 1 instead (the previous item's last drain, done in its epilogue):
        // by then the phase of pair g - 2 may already lie two completions back, which a parity wait cannot tell
        // from "not yet".
        auto s_buffer_free = [&](int n) -> bool {
          const uint32_t g = g_base + n;
          if (n == 0) return g < 1 || mbar_wait_idle(dq_drained, (g - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          return g < 2 || mbar_wait_idle(dq_drained, (g - 2) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
        };
        // ---- item prologue: K / V of the previous item are no longer read once its last MMAs retired
        if (items > 0 && !mbar_wait_idle(done, (items - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
        mbar_arrive_expect_tx(kv_full, 2 * S::TILE);
        load_tile<D>(smem + S::OFF_K, &tmap_k, kv_full, itm.k0, itm.hk, itm.b);
        load_tile<D>(smem + S::OFF_V, &tmap_v, kv_full, itm.k0, itm.hk, itm.b);
        ok = load_q(0);
        if (ok && n_it > 1) ok = load_q(1);
        ok = ok && mbar_wait_idle(kv_full, items & 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER) &&
             mbar_wait_idle(&qdo_full[g_base % QS], (g_base / QS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) && s_buffer_free(0);
        if (!ok) break;
        tc_fence_after();
        issue_S(0);
        issue_dP(0);   // dP(previous pair) was read before that pair's pds_full, which this thread has waited for
        for (int it = 0; it < n_it && ok; ++it) {
          const uint32_t g = g_base + it;
          if (it + 1 < n_it) {  // S of the next pair while the softmax warps work on this one
            ok = mbar_wait_idle(&qdo_full[(g + 1) % QS], ((g + 1) / QS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) && s_buffer_free(it + 1);
            if (!ok) break;
            tc_fence_after();
            issue_S(it + 1);
          }
          if (it + 2 < n_it && !load_q(it + 2)) { ok = false; break; }
          if (!mbar_wait_idle(pds_full, g & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) { ok = false; break; }
          // the first dV / dK MMA of an item overwrites the accumulators: the previous item's epilogue must have read them
          if (it == 0 && items > 0 && !mbar_wait_idle(acc_free, (items - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const int s = g % QS;
          const uint32_t aQ = smem_u32(smem + S::OFF_Q + s * S::TILE);
          const uint32_t aDO = smem_u32(smem + S::OFF_DO + s * S::TILE);
          // dQ_partial first (the softmax warps drain it early in the next pair), over the scores of this pair
#pragma unroll
          for (int kk = 0; kk < ATT_BN / 16; ++kk)
            umma_f16_ss(tmem_S0 + (g & 1) * 128, stage_desc_kmajor(aDS, kk), tile_desc_mnmajor<D>(aK, kk), idesc_Q, kk > 0 ? 1u : 0u);
          umma_commit(dq_full);
          if (it + 1 < n_it) issue_dP(it + 1);  // ahead of dV / dK: the softmax warps of the next pair need it first
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
        g_base += n_it;
        ++items;
      }
    }
  } else {
    // ================================================================== softmax warps
    // warps 0..3 take score columns 0..63, warps 4..7 columns 64..127 of the same 128 rows
    const int quarter = warp & 3, chalf = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint8_t* sP = smem + S::OFF_P;
    uint8_t* sDS = smem + S::OFF_DS;
    bool ok = true;
    uint32_t g_base = 0, items = 0;
    // dQ_partial of pair g (query tile starting at row q0 of head h): each warp owns a 32-row x 32-column block.  It
    // goes TMEM -> registers -> the warp's own swizzled fp32 staging block -> ONE TMA reduce-add into the accumulation
    // buffer (full 128-byte lines through the copy engine instead of 32 scattered 16-byte atomics per instruction).
    uint8_t* dq_stage = smem + S::OFF_DQ + warp * 4096;
    auto drain_dq = [&](uint32_t g, int bq, int h, int q0) -> bool {
      if (!mbar_wait(dq_full, g & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) return false;
      tc_fence_after();
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32b_x32(tmem_S0 + (g & 1) * 128 + lane_sel + chalf * 32, r);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_drained);
      if (lane == 0) bulk_wait_group_read<0>();   // the previous reduce of this warp has read the staging block
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float4 v4 = make_float4(__uint_as_float(r[c * 4]) * p.scale, __uint_as_float(r[c * 4 + 1]) * p.scale,
                                __uint_as_float(r[c * 4 + 2]) * p.scale, __uint_as_float(r[c * 4 + 3]) * p.scale);
        *reinterpret_cast<float4*>(dq_stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = v4;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_reduce_add_4d(&tmap_dq, dq_stage, chalf * 32, q0 + quarter * 32, h, bq);   // rows past Tq are clipped
        bulk_commit_group();
      }
      return true;
    };
    for (int k = 0; ok; ++k) {
      FbItem itm;
      if (!fb_item(k, p, itm)) break;
      const int kr = itm.k0 + row;
      const uint32_t src = chalf == 0 ? tmem_dV : tmem_dK;  // column half 0 writes dV, half 1 writes dK
      const float mul = chalf == 0 ? 1.f : p.scale;
      __nv_bfloat16* dst = chalf == 0 ? p.dv + (long long)itm.b * p.dv_sb + (long long)kr * p.dv_st + (long long)itm.hk * p.dv_sh
                                      : p.dk + (long long)itm.b * p.dk_sb + (long long)kr * p.dk_st + (long long)itm.hk * p.dk_sh;
      if (itm.n_it == 0) {  // no query row sees this key tile: zero gradients
        if (kr < p.Tk) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      const int n_it = itm.n_it;
      int prev_h = 0, prev_qi = 0;
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t g = g_base + it;
        const int h = itm.hk * group + it / itm.per_head;
        const int qi = (itm.i_start + it % itm.per_head) * ATT_BM + row;
        const bool row_ok = qi < p.Tq;
        const long long sidx = ((long long)itm.b * p.H + h) * p.Tq + qi;
        const float lse2 = row_ok ? p.lse[sidx] * 1.4426950408889634f : 0.f;
        const float dl = row_ok ? p.delta[sidx] : 0.f;
        const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);
        if (!mbar_wait(&s_full[g & 1], (g >> 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        uint32_t rs[2][32], rp[2][32];
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_S0 + (g & 1) * 128 + lane_sel + (chalf * 2 + u) * 32, rs[u]);
        tmem_ld_wait();
        // probabilities first (they only need S); rs is reused for them
        const bool partial = (p.causal && itm.k0 + ATT_BN - 1 > (qi - row) + off) || (itm.k0 + ATT_BN > p.Tk) || (qi - row + ATT_BM > p.Tq);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int c = chalf * 2 + u;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float e = ex2_approx(fmaf(__uint_as_float(rs[u][i]), p.scale_log2, -lse2));
            if (partial && !(row_ok && (itm.k0 + c * 32 + i <= limit))) e = 0.f;
            rs[u][i] = __float_as_uint(e);
          }
        }
        // dQ_partial of the previous pair (issued first after that pair's staging) is complete by now
        if (it > 0 && !drain_dq(g - 1, itm.b, prev_h, prev_qi)) { ok = false; break; }
        prev_h = h;
        prev_qi = qi - row;
        if (!mbar_wait(dp_full, g & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 2; ++u) tmem_ld_32x32b_x32(tmem_dP + lane_sel + (chalf * 2 + u) * 32, rp[u]);
        tmem_ld_wait();
        // P / dS staging is read by the dV / dK / dQ MMAs of the previous pair until they retire
        if (g > 0 && !mbar_wait(pds_empty, (g - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
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
      if (!ok) break;
      // ---- item epilogue: last dQ_partial, then dK / dV of this key tile
      if (!drain_dq(g_base + n_it - 1, itm.b, prev_h, prev_qi)) { ok = false; break; }
      if (!mbar_wait(done, items & 1, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(src + lane_sel + c * 32, r);
        tmem_ld_wait();
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
      mbar_arrive(acc_free);
      g_base += n_it;
      ++items;
    }
  }

  __syncwarp();
  if (warp != FB_CTRL_WARP && lane == 0) bulk_wait_group<0>();   // this warp's dQ reduces have landed
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == FB_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// dq[b][t][h][:] (bf16, strided) = dq_acc[b][t][h][:] (fp32, contiguous); 8 elements per thread.
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n8, int H, int Tq,
                                       long long sb, long long st, long long sh) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const long long e = i * 8;
  const int d = int(e % FB_D);
  const long long row = e / FB_D;  // (b * Tq + t) * H + h
  const int h = int(row % H);
  const long long bt = row / H;
  const int t = int(bt % Tq);
  const long long b = bt / Tq;
  const float4 x = *reinterpret_cast<const float4*>(acc + e), y = *reinterpret_cast<const float4*>(acc + e + 4);
  uint4 w;
  w.x = pack_bf16x2(x.x, x.y);
  w.y = pack_bf16x2(x.z, x.w);
  w.z = pack_bf16x2(y.x, y.y);
  w.w = pack_bf16x2(y.z, y.w);
  *reinterpret_cast<uint4*>(dq + b * sb + t * st + h * sh + d) = w;
}

// Longest-first assignment of (key tile, kv head, batch) items to CTAs, cached on the device per geometry.
namespace {
struct FbKey {
  int device, B, H, Hkv, Tq, Tk, causal, grid;
  bool operator<(const FbKey& o) const {
    return std::tie(device, B, H, Hkv, Tq, Tk, causal, grid) < std::tie(o.device, o.B, o.H, o.Hkv, o.Tq, o.Tk, o.causal, o.grid);
  }
};
struct FbList {
  int* dev = nullptr;
  int per_cta = 0;
};
FbList fb_item_list(const AttnArgs& a, int grid, int device, cudaStream_t stream) {
  static std::mutex mu;
  static std::map<FbKey, FbList> cache;
  std::lock_guard<std::mutex> lock(mu);
  const FbKey key{device, a.B, a.H, a.Hkv, a.Tq, a.Tk, a.causal, grid};
  auto f = cache.find(key);
  if (f != cache.end()) return f->second;
  const int n_kv = (a.Tk + ATT_BN - 1) / ATT_BN, n_q = (a.Tq + ATT_BM - 1) / ATT_BM, group = a.H / a.Hkv;
  std::vector<std::pair<int, int>> items;  // (cost, id)
  for (int bh = 0; bh < a.B * a.Hkv; ++bh)
    for (int j = 0; j < n_kv; ++j) {
      const int i_start = a.causal ? std::max(0, j * ATT_BN - (a.Tk - a.Tq)) / ATT_BM : 0;
      const int cost = std::max(0, n_q - i_start) * group + 1;  // + 1: K / V load, pipeline fill and the dK / dV epilogue
      items.emplace_back(cost, bh * n_kv + j);
    }
  std::stable_sort(items.begin(), items.end(), [](const auto& x, const auto& y) { return x.first > y.first; });
  std::vector<std::vector<int>> per(grid);
  using Load = std::pair<long long, int>;
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int c = 0; c < grid; ++c) heap.emplace(0, c);
  for (const auto& it : items) {
    Load top = heap.top();
    heap.pop();
    per[top.second].push_back(it.second);
    heap.emplace(top.first + it.first, top.second);
  }
  size_t mx = 1;
  for (const auto& v : per) mx = std::max(mx, v.size());
  std::vector<int> flat(size_t(grid) * mx, -1);
  for (int c = 0; c < grid; ++c) std::copy(per[c].begin(), per[c].end(), flat.begin() + size_t(c) * mx);
  FbList out;
  out.per_cta = int(mx);
  RT_CUDA_CHECK(cudaMalloc(&out.dev, flat.size() * sizeof(int)));
  RT_CUDA_CHECK(cudaMemcpyAsync(out.dev, flat.data(), flat.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
  RT_CUDA_CHECK(cudaStreamSynchronize(stream));  // `flat` is pageable host memory that dies with this scope
  cache.emplace(key, out);
  return out;
}
}  // namespace

// Backward for D == 64 with a caller-provided fp32 accumulation buffer a.dq_acc [B][Tq][H][64].  a.delta must already
// hold rowsum(o * do) (attn_bwd computes it before calling this).
void attn_bwd_fused_d64(const AttnArgs& a, cudaStream_t stream) {
  using S = FusedBwdSmem;
  const int device = current_device();
  static bool configured[64] = {false};
  if (!configured[device]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device] = true;
  }
  constexpr int D = FB_D;
  CUtensorMap tq = make_tmap_2byte_4d(a.q, D, a.Tq, a.H, a.B, a.q_st, a.q_sh, a.q_sb, 64, 128);
  CUtensorMap tk = make_tmap_2byte_4d(a.k, D, a.Tk, a.Hkv, a.B, a.k_st, a.k_sh, a.k_sb, 64, 128);
  CUtensorMap tv = make_tmap_2byte_4d(a.v, D, a.Tk, a.Hkv, a.B, a.v_st, a.v_sh, a.v_sb, 64, 128);
  CUtensorMap tdo = make_tmap_2byte_4d(a.d_o, D, a.Tq, a.H, a.B, a.o_st, a.o_sh, a.o_sb, 64, 128);
  // fp32 accumulation buffer [B][Tq][H][64] seen as (d, t, h, b); one reduce covers 32 columns x 32 rows
  CUtensorMap tdq = make_tmap_f32_4d(a.dq_acc, D, a.Tq, a.H, a.B, uint64_t(a.H) * D, D, uint64_t(a.Tq) * a.H * D, 32, 32);
  AttnBwdFusedParams p{};
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
  p.dq_acc = a.dq_acc;
  p.dk = reinterpret_cast<__nv_bfloat16*>(a.dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(a.dv);
  p.dk_sb = a.dk_sb; p.dk_st = a.dk_st; p.dk_sh = a.dk_sh;
  p.dv_sb = a.dv_sb; p.dv_st = a.dv_st; p.dv_sh = a.dv_sh;
  p.n_kv_tiles = (a.Tk + ATT_BN - 1) / ATT_BN;
  p.status = status_word(device);
  const long long n_acc = (long long)a.B * a.Tq * a.H * D;
  RT_CUDA_CHECK(cudaMemsetAsync(a.dq_acc, 0, size_t(n_acc) * sizeof(float), stream));
  const int total_items = a.B * a.Hkv * p.n_kv_tiles;
  const int grid = std::min(total_items, sm_count(device));
  const FbList il = fb_item_list(a, grid, device, stream);
  p.item_list = il.dev;
  p.items_per_cta = il.per_cta;
  attn_bwd_fused_kernel<<<grid, FB_THREADS, S::TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);
  RT_LAUNCH_CHECK();
  const long long n8 = n_acc / 8;
  attn_dq_convert_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(a.dq_acc, reinterpret_cast<__nv_bfloat16*>(a.dq), n8, a.H, a.Tq,
                                                                         a.dq_sb, a.dq_st, a.dq_sh);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
