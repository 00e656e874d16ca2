// Flash-attention forward, persistent ping-pong form (sm_100a): causal / non-causal, MHA and GQA, head dim 64 or
// 128, bf16 or fp16 in, fp32 softmax statistics, 16-bit out + fp32 log-sum-exp.
//
// One CTA per SM walks a list of work items; an item is TWO adjacent 128-row query tiles of one (batch, head) and
// the key tiles they see.  Items are ordered longest first (causal: the bottom query rows) and dealt to the CTAs in
// serpentine order, so the per-CTA totals differ by a few key tiles and no CTA pays a prologue per query tile.
//
// Warp roles (352 threads):
//   warps 0-3 / 4-7  softmax group of query tile 0 / 1: thread t owns score row t (tcgen05.ld hands TMEM lane t to
//                    thread t of the group), so row max / row sum need no shuffles
//   warp 8 / 9       lane 0 issues every tcgen05.mma of tile 0 / 1
//   warp 10          lane 0 issues every TMA load; the warp owns the TMEM allocation
// Tensor memory (512 columns): S0 | S1 | O0 | O1 (| P0 | P1 for D = 64; for D = 128 P_i overlays S_i).
//   S_i = Q_i K_j^T                      SS-form MMA, fp32 in TMEM
//   softmax group i: S row -> registers, running reference maximum, exp2, P row packed to 16 bit and written back
//                    to TENSOR MEMORY (tcgen05.st): no shared-memory staging, no proxy fence
//   O_i += P_i V_j                       TS-form MMA (A = P from TMEM, B = V from shared memory)
// While group 0 exponentiates S0(j), the tensor core produces S1(j) and O1 += P1 V(j-1) and vice versa.  For D = 64
// S_i(j+1) is issued as soon as group i holds S_i(j) in registers; for D = 128 (P overlays S) right after
// O_i += P_i V_j.  The reference maximum is only raised (and O rescaled through a TMEM load-scale-store) when a row's
// block maximum exceeds it by more than 2^8; until then exponentials are taken against the stale maximum, which the
// final division by the row sum cancels exactly.  K and V tiles stream through TMA rings shared by both query tiles.
// The score matrix never reaches HBM, unlike the reference, which materialises [B,H,T,T] scores
// (src/nn/transformer_phase6.rs:342-374) and whose "fused_attention" kernel string is never compiled
// (src/gpu/custom_kernels.rs:439-536).
#include "../api.h"
#include "../common/launch.h"
#include "attn_common.cuh"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <vector>

namespace rt {

struct AttnFwdPPParams {
  int B, H, Hkv, Tq, Tk;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  uint16_t* o;       // bf16, or fp16 in the F16 instantiation
  long long o_sb, o_st, o_sh;
  float* lse;  // [B][H][Tq]
  int n_pairs;  // pairs of query tiles per (batch, head)
  int total_items;
  const int* item_list;  // [gridDim.x][items_per_cta]: the items of each CTA in processing order, -1 = none
  int items_per_cta;
  int* status;
#ifdef RT_ATTN_PROF
  long long* prof;  // [gridDim.x][2 groups][8]: cycles spent in each phase by lane 0 of the group's first warp
#endif
};

template <int D>
struct AttnFwdPPSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int KV_STAGES = (D == 64) ? 4 : 2;
  static constexpr int OFF_Q = 0;                       // two query tiles
  static constexpr int OFF_K = 2 * TILE;
  static constexpr int OFF_V = OFF_K + KV_STAGES * TILE;
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * TILE;
  // q_full[2] q_empty[2] s_full[2] s_free[2] p_full[2] pv_done[2] o_free[2] k_full[KS] k_empty[KS] v_full[KS] v_empty[KS]
  static constexpr int N_BARS = 16 + 4 * KV_STAGES;   // ... + tok[2]
  static constexpr int TOTAL = OFF_BAR + N_BARS * 8 + 16;
  static_assert(TOTAL <= 232448, "attention: shared memory over the per-CTA limit");
};

#ifdef RT_ATTN_PROF
long long*& attn_prof_buffer() {
  static long long* b = nullptr;
  return b;
}
extern "C" long long* rt_attn_prof_buffer() { return attn_prof_buffer(); }
#endif

constexpr float ATT_PP_RESCALE_THRESHOLD = 8.f;  // log2 units
// The CTA owns 384 x 168 = 64512 registers at launch; the two budgets must fit into that or setmaxnreg.inc never returns.
constexpr int ATT_PP_REGS_CONTROL = 64, ATT_PP_REGS_SOFTMAX = 216;  // 128 x 64 + 256 x 216 = 63488
static_assert(128 * ATT_PP_REGS_CONTROL + 256 * ATT_PP_REGS_SOFTMAX <= 384 * 168, "register budgets exceed the CTA allocation");
constexpr int ATT_PP_THREADS = 384;  // 12 warps; warp 11 idles (register re-division works on groups of four warps)

// 2^x for x <= ~8 on the FMA / integer pipes: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a degree-3
// minimax polynomial (relative error 7.7e-5, far below the 16-bit rounding of P), then n is added to the exponent
// field.  Used for one exponential in eight so that the special-function unit (16 ex2 per clock and SM) and the FMA
// pipe finish a score tile at about the same time.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float t = x + 12582912.f;                 // 1.5 * 2^23: the integer part of x lands in the low mantissa bits
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.05511089786887169f, 0.2426059991121292f);
  p = fmaf(p, f, 0.6932721734046936f);
  p = fmaf(p, f, 0.9999287128448486f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Item id = pair * (B * H) + batch * H + head.
__device__ __forceinline__ void pp_decode_item(int w, const AttnFwdPPParams& p, int& b, int& h, int& pair) {
  const int bh = p.B * p.H;
  pair = w / bh;
  const int r = w - pair * bh;
  b = r / p.H;
  h = r - b * p.H;
}
// k-th item of this CTA; -1 past the end.  The host deals the items longest first to the least loaded CTA, so the
// per-CTA totals differ by less than one short item (see build_item_list).
__device__ __forceinline__ int pp_item_of(int k, const AttnFwdPPParams& p) {
  return k < p.items_per_cta ? __ldg(p.item_list + (long long)blockIdx.x * p.items_per_cta + k) : -1;
}
// Number of key tiles query tile `qt` looks at (0: the tile has no rows or sees no key).
__device__ __forceinline__ int pp_n_kv(int qt, const AttnFwdPPParams& p) {
  const int q0 = qt * ATT_BM;
  if (q0 >= p.Tq) return 0;
  int n = (p.Tk + ATT_BN - 1) / ATT_BN;
  if (p.causal) {
    const int last_col = min(p.Tk - 1, q0 + ATT_BM - 1 + (p.Tk - p.Tq));
    n = last_col < 0 ? 0 : min(n, last_col / ATT_BN + 1);
  }
  return n;
}

template <int D, bool F16, int POLY>
__global__ void __launch_bounds__(ATT_PP_THREADS, 1)
attn_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const AttnFwdPPParams p) {
  pdl_launch_dependents();  // a dependent-launch kernel that follows may set up while this one runs
  using S = AttnFwdPPSmem<D>;
  constexpr int KS = S::KV_STAGES;
  constexpr bool ALIAS = (D == 128);  // P_i overlays S_i
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 2;
  uint64_t* s_full = bars + 4;
  uint64_t* s_free = bars + 6;
  uint64_t* p_full = bars + 8;
  uint64_t* pv_done = bars + 10;
  uint64_t* o_free = bars + 12;
  uint64_t* k_full = bars + 14;
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* tok = v_empty + KS;  // D = 128 only: the two MMA issuers take turns, tile 0 first
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S::N_BARS);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_free[i], 128);
      mbar_init(&tok[i], 1);
    }
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
    }
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 10) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_S = [&](int i) { return tmem_base + uint32_t(i) * 128u; };
  auto tmem_O = [&](int i) { return tmem_base + 256u + uint32_t(i) * uint32_t(D); };
  auto tmem_P = [&](int i) { return ALIAS ? tmem_S(i) : (tmem_base + 384u + uint32_t(i) * 64u); };
  const int group = p.H / p.Hkv;

  if (warp >= 8) {
  // Control warps give registers up, the softmax groups take them (setmaxnreg acts on aligned groups of four warps).
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ATT_PP_REGS_CONTROL));
  if (warp == 10) {
    // ================================================================== TMA producer
    if (lane == 0) {
      uint32_t kv_it = 0;            // key / value tiles loaded so far (ring position)
      uint32_t q_items[2] = {0, 0};  // items in which tile i was active so far
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int w = pp_item_of(k, p);
        if (w < 0) break;
        int b, h, pair;
        pp_decode_item(w, p, b, h, pair);
        const int hk = h / group;
        const int n0 = pp_n_kv(2 * pair, p), n1 = pp_n_kv(2 * pair + 1, p);
        const int n = max(n0, n1);
        // Order: the first active query tile, the first key / value tile, then the other query tile and the rest, so
        // that the group that finished the previous item first is not held up by the other group's last tile.
        auto load_q = [&](int i) -> bool {
          if ((i == 0 ? n0 : n1) == 0) return true;
          if (q_items[i] > 0 && !mbar_wait_idle(&q_empty[i], (q_items[i] - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
          mbar_arrive_expect_tx(&q_full[i], S::TILE);
          load_tile<D>(smem + S::OFF_Q + i * S::TILE, &tmap_q, &q_full[i], (2 * pair + i) * ATT_BM, h, b);
          ++q_items[i];
          return true;
        };
        auto load_kv = [&](int j) -> bool {
          const int s = kv_it % KS;
          const uint32_t ph = (kv_it / KS) & 1;
          if (!mbar_wait_idle(&k_empty[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
          mbar_arrive_expect_tx(&k_full[s], S::TILE);
          load_tile<D>(smem + S::OFF_K + s * S::TILE, &tmap_k, &k_full[s], j * ATT_BN, hk, b);
          if (!mbar_wait_idle(&v_empty[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) return false;
          mbar_arrive_expect_tx(&v_full[s], S::TILE);
          load_tile<D>(smem + S::OFF_V + s * S::TILE, &tmap_v, &v_full[s], j * ATT_BN, hk, b);
          ++kv_it;
          return true;
        };
        const int first = n0 > 0 ? 0 : 1;
        ok = load_q(first);
        if (ok && n > 0) ok = load_kv(0);
        if (ok) ok = load_q(1 - first);
        for (int j = 1; j < n && ok; ++j) ok = load_kv(j);
      }
    }
  } else if (warp < 10) {
    // ================================================================== MMA issuer of query tile i
    const int i = warp - 8;
    if (lane == 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, !F16);
      constexpr uint32_t idesc_PV = make_idesc_f16(128, D, false, true, !F16);
      const uint32_t aQ = smem_u32(smem + S::OFF_Q + i * S::TILE);
      uint32_t kv_it = 0;   // ring position at the start of the current item
      uint32_t cnt = 0;     // key tiles this query tile has processed over all items (phase of the per-tile barriers)
      uint32_t items = 0;   // items in which this tile was active
      uint32_t slot = 0;    // key-tile slots walked so far (both issuers walk the same number per item)
      bool ok = true;
      // D = 128 (P overlays S): the two issuers alternate strictly, tile 0 then tile 1, per key tile.  Tile 1's
      // "O += P V, next S" batch then always follows tile 0's, which keeps the two softmax groups half a period apart:
      // one exponentiates while the tensor core works for the other, instead of both waiting for it at once.
      auto turn_acquire = [&]() -> bool {
        if (!ALIAS) return true;
        if (i == 0) return slot == 0 || mbar_wait_idle(&tok[0], (slot - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
        return mbar_wait_idle(&tok[1], slot & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
      };
      auto turn_release = [&]() {
        if (ALIAS) mbar_arrive(&tok[1 - i]);
        ++slot;
      };
      auto issue_S = [&](uint32_t ring_pos) {
        const int s = ring_pos % KS;
        const uint32_t aK = smem_u32(smem + S::OFF_K + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S(i), tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[i]);
        umma_commit(&k_empty[s]);
      };
      for (int k = 0; ok; ++k) {
        const int w = pp_item_of(k, p);
        if (w < 0) break;
        int b, h, pair;
        pp_decode_item(w, p, b, h, pair);
        const int n0 = pp_n_kv(2 * pair, p), n1 = pp_n_kv(2 * pair + 1, p);
        const int n = max(n0, n1);
        const int ni = i == 0 ? n0 : n1;
        if (ni > 0) {
          // first S of the item: Q_i and K(0) loaded, the S region free of the previous item's last tile
          ok = mbar_wait_idle(&q_full[i], items & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) &&
               mbar_wait_idle(&k_full[kv_it % KS], (kv_it / KS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (ok && !ALIAS && cnt > 0) ok = mbar_wait_idle(&s_free[i], (cnt - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_S(kv_it);
          if (ni == 1) umma_commit(&q_empty[i]);
        }
        for (int j = 0; j < ni && ok; ++j, ++cnt) {
          const uint32_t pos = kv_it + j;
          const int s = pos % KS;
          const uint32_t ph = (pos / KS) & 1;
          if (!ALIAS && j + 1 < ni) {  // next S while this tile's softmax runs: needs S(j) in registers and K(j+1)
            ok = mbar_wait_idle(&s_free[i], cnt & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) &&
                 mbar_wait_idle(&k_full[(pos + 1) % KS], ((pos + 1) / KS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            issue_S(pos + 1);
            if (j + 2 == ni) umma_commit(&q_empty[i]);
          }
          ok = turn_acquire() && mbar_wait_idle(&p_full[i], cnt & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) &&
               mbar_wait_idle(&v_full[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (ok && j == 0 && items > 0) ok = mbar_wait_idle(&o_free[i], (items - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          const uint32_t aV = smem_u32(smem + S::OFF_V + s * S::TILE);
#pragma unroll
          for (int kk = 0; kk < ATT_BN / 16; ++kk)
            umma_f16_ts(tmem_O(i), tmem_P(i) + kk * 8, tile_desc_mnmajor<D>(aV, kk), idesc_PV, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&pv_done[i]);
          umma_commit(&v_empty[s]);
          if (ALIAS && j + 1 < ni) {  // P overlays S: the next S follows O += P V in issue order
            if (!mbar_wait_idle(&k_full[(pos + 1) % KS], ((pos + 1) / KS) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
            issue_S(pos + 1);
            if (j + 2 == ni) umma_commit(&q_empty[i]);
          }
          turn_release();
        }
        // key tiles only the other query tile looks at: hand the ring slots back once they are loaded
        for (int j = ni; j < n && ok; ++j) {
          const uint32_t pos = kv_it + j;
          const int s = pos % KS;
          const uint32_t ph = (pos / KS) & 1;
          ok = turn_acquire() && mbar_wait_idle(&k_full[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (ok) mbar_arrive(&k_empty[s]);
          ok = ok && mbar_wait_idle(&v_full[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (ok) mbar_arrive(&v_empty[s]);
          if (ok) turn_release();
        }
        kv_it += n;
        if (ni > 0) ++items;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ATT_PP_REGS_SOFTMAX));
    // ================================================================== softmax group of query tile i
    const int i = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
    const int off = p.Tk - p.Tq;  // causal: key col visible iff col <= row + off
    uint32_t cnt = 0;
    bool ok = true;
#ifdef RT_ATTN_PROF
    long long pf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long t_prev = clock64();
#define PROF_MARK(slot) { const long long t_now = clock64(); pf[slot] += t_now - t_prev; t_prev = t_now; }
#else
#define PROF_MARK(slot)
#endif
    for (int k = 0; ok; ++k) {
      const int w = pp_item_of(k, p);
      if (w < 0) break;
      int b, h, pair;
      pp_decode_item(w, p, b, h, pair);
      const int qt = 2 * pair + i;
      const int q0 = qt * ATT_BM;
      const int qi = q0 + row;
      const int ni = pp_n_kv(qt, p);
      uint16_t* orow = p.o + (long long)b * p.o_sb + (long long)qi * p.o_st + (long long)h * p.o_sh;
      if (ni == 0) {  // no visible key: zero output, -inf log-sum-exp
        if (qi < p.Tq) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0u, 0u, 0u, 0u);
          p.lse[((long long)b * p.H + h) * p.Tq + qi] = -INFINITY;
        }
        continue;
      }
      const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);  // last visible column
      float m = 0.f, l = 0.f;
      for (int j = 0; j < ni && ok; ++j, ++cnt) {
        PROF_MARK(0)
        if (!mbar_wait(&s_full[i], cnt & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        PROF_MARK(1)
        uint32_t r[128];
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tmem_ld_32x32b_x32(tmem_S(i) + lane_sel + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_ld_wait();
        PROF_MARK(2)
        if (!ALIAS) {
          tc_fence_before();
          mbar_arrive(&s_free[i]);  // S is in registers: the next S MMA may overwrite TMEM now
        }
        const int col_base = j * ATT_BN;
        const bool partial = (p.causal && col_base + ATT_BN - 1 > q0 + off) || (col_base + ATT_BN > p.Tk);
        if (partial) {
#pragma unroll
          for (int e = 0; e < 128; ++e)
            if (col_base + e > limit) r[e] = 0xff800000u;  // -inf
        }
        float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;   // four independent chains
#pragma unroll
        for (int e = 0; e < 128; e += 8) {
          a0 = fmax3(a0, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
          a1 = fmax3(a1, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
          a2 = fmax3(a2, __uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
          a3 = fmax3(a3, __uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
        }
        const float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) * p.scale_log2;  // scale > 0: max commutes with it
        float alpha = 1.f;
        bool rescale = false;
        if (j == 0) {
          m = (mx == -INFINITY) ? 0.f : mx;
        } else {
          rescale = __any_sync(0xffffffffu, mx > m + ATT_PP_RESCALE_THRESHOLD);
          if (rescale) {
            const float m_new = fmaxf(m, mx);
            alpha = ex2_approx(m - m_new);
            m = m_new;
            l *= alpha;
          }
        }
        PROF_MARK(7)
        const float neg_m = -m;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        uint32_t pk[64];
#pragma unroll
        for (int e = 0; e < 128; e += 4) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(r[e]), p.scale_log2, neg_m));
          const float e1 = ex2_approx(fmaf(__uint_as_float(r[e + 1]), p.scale_log2, neg_m));
          const float e2 = ex2_approx(fmaf(__uint_as_float(r[e + 2]), p.scale_log2, neg_m));
          const float x3 = fmaf(__uint_as_float(r[e + 3]), p.scale_log2, neg_m);
          const float e3 = (POLY == 4 || (POLY == 8 && (e & 4))) ? exp2_poly(x3) : ex2_approx(x3);
          sum0 += e0;
          sum1 += e1;
          sum2 += e2;
          sum3 += e3;
          pk[e / 2] = pack_2x16<F16>(e0, e1);
          pk[e / 2 + 1] = pack_2x16<F16>(e2, e3);
        }
        l += (sum0 + sum1) + (sum2 + sum3);
        PROF_MARK(3)
        // O_i += P V of the previous key tile must have retired before P is overwritten or O rescaled
        if (cnt > 0 && !mbar_wait(&pv_done[i], (cnt - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        PROF_MARK(4)
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            __syncwarp();
            tmem_ld_32x32b_x32(tmem_O(i) + lane_sel + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32b_x32(tmem_O(i) + lane_sel + c * 32, o);
          }
        }
        __syncwarp();
        tmem_st_32x32b_x32(tmem_P(i) + lane_sel, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st_32x32b_x32(tmem_P(i) + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[i]);
        PROF_MARK(5)
      }
      // ---- epilogue of the item: O / l -> global, log-sum-exp, then hand O back to the MMA warp
      if (ok) ok = mbar_wait(&pv_done[i], (cnt - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
      if (!ok) break;
      tc_fence_after();
      PROF_MARK(6)
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool wide_store = ((reinterpret_cast<uintptr_t>(orow) & 31) == 0);   // rows of this (batch, head) 32-byte aligned
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_O(i) + lane_sel + c * 32, o);
        tmem_ld_wait();
        if (qi < p.Tq) {
          uint32_t w16[16];
#pragma unroll
          for (int q = 0; q < 16; ++q)
            w16[q] = pack_2x16<F16>(__uint_as_float(o[2 * q]) * inv, __uint_as_float(o[2 * q + 1]) * inv);
          if (wide_store) {  // 32-byte stores: two per 32 columns
            st_global_v8(orow + c * 32, *reinterpret_cast<uint32_t(*)[8]>(&w16[0]));
            st_global_v8(orow + c * 32 + 16, *reinterpret_cast<uint32_t(*)[8]>(&w16[8]));
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              reinterpret_cast<uint4*>(orow + c * 32)[q] = make_uint4(w16[q * 4], w16[q * 4 + 1], w16[q * 4 + 2], w16[q * 4 + 3]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&o_free[i]);
      if (qi < p.Tq)
        p.lse[((long long)b * p.H + h) * p.Tq + qi] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      PROF_MARK(7)
    }
#ifdef RT_ATTN_PROF
    if ((warp & 3) == 0 && lane == 0 && p.prof)
      for (int e = 0; e < 8; ++e) p.prof[(blockIdx.x * 2 + i) * 8 + e] = pf[e];
#endif
  }

  // Common exit: on abort give in-flight bulk copies time to land, then release TMEM.
  __syncwarp();
  if (ctl->abort) {
    for (int it = 0; it < 200; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Longest-processing-time-first assignment of the work items to `grid` CTAs, cached on the device per problem
// geometry.  The cost of an item is the number of key tiles its two query tiles look at; items go, longest first, to
// the CTA with the smallest total so far, and each CTA processes its own items longest first.
struct ItemListKey {
  int device, B, H, Tq, Tk, causal, grid;
  bool operator<(const ItemListKey& o) const {
    return std::tie(device, B, H, Tq, Tk, causal, grid) < std::tie(o.device, o.B, o.H, o.Tq, o.Tk, o.causal, o.grid);
  }
};
struct ItemList {
  int* dev = nullptr;
  int per_cta = 0;
};
static ItemList build_item_list(const AttnArgs& a, int n_pairs, int grid, int device, cudaStream_t stream) {
  static std::mutex mu;
  static std::map<ItemListKey, ItemList> cache;
  std::lock_guard<std::mutex> lock(mu);
  const ItemListKey key{device, a.B, a.H, a.Tq, a.Tk, a.causal, grid};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  const int bh = a.B * a.H;
  auto n_kv = [&](int qt) {
    const int q0 = qt * ATT_BM;
    if (q0 >= a.Tq) return 0;
    int n = (a.Tk + ATT_BN - 1) / ATT_BN;
    if (a.causal) {
      const int last_col = std::min(a.Tk - 1, q0 + ATT_BM - 1 + (a.Tk - a.Tq));
      n = last_col < 0 ? 0 : std::min(n, last_col / ATT_BN + 1);
    }
    return n;
  };
  std::vector<std::pair<int, int>> items;  // (cost, id)
  items.reserve(size_t(n_pairs) * bh);
  for (int pair = 0; pair < n_pairs; ++pair) {
    const int cost = n_kv(2 * pair) + n_kv(2 * pair + 1) + 1;  // + 1: per-item prologue / epilogue
    for (int r = 0; r < bh; ++r) items.emplace_back(cost, pair * bh + r);
  }
  std::stable_sort(items.begin(), items.end(), [](const auto& x, const auto& y) { return x.first > y.first; });
  std::vector<std::vector<int>> per(grid);
  using Load = std::pair<long long, int>;  // (total cost, cta)
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int c = 0; c < grid; ++c) heap.emplace(0, c);
  for (const auto& itx : items) {
    Load top = heap.top();
    heap.pop();
    per[top.second].push_back(itx.second);
    heap.emplace(top.first + itx.first, top.second);
  }
  size_t mx = 1;
  for (const auto& v : per) mx = std::max(mx, v.size());
  std::vector<int> flat(size_t(grid) * mx, -1);
  for (int c = 0; c < grid; ++c) std::copy(per[c].begin(), per[c].end(), flat.begin() + size_t(c) * mx);
  ItemList out;
  out.per_cta = int(mx);
  RT_CUDA_CHECK(cudaMalloc(&out.dev, flat.size() * sizeof(int)));
  RT_CUDA_CHECK(cudaMemcpyAsync(out.dev, flat.data(), flat.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
  RT_CUDA_CHECK(cudaStreamSynchronize(stream));  // `flat` is pageable host memory that dies with this scope
  cache.emplace(key, out);
  return out;
}

template <int D, bool F16, int POLY>
static void launch_fwd_pp(const AttnArgs& a, cudaStream_t stream) {
  using S = AttnFwdPPSmem<D>;
  const int device = current_device();
  auto kern = attn_fwd_pp_kernel<D, F16, POLY>;
  static bool configured[64] = {false};
  if (!configured[device]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device] = true;
  }
  CUtensorMap tq = make_tmap_2byte_4d(a.q, D, a.Tq, a.H, a.B, a.q_st, a.q_sh, a.q_sb, 64, 128);
  CUtensorMap tk = make_tmap_2byte_4d(a.k, D, a.Tk, a.Hkv, a.B, a.k_st, a.k_sh, a.k_sb, 64, 128);
  CUtensorMap tv = make_tmap_2byte_4d(a.v, D, a.Tk, a.Hkv, a.B, a.v_st, a.v_sh, a.v_sb, 64, 128);
  AttnFwdPPParams p{};
  p.B = a.B;
  p.H = a.H;
  p.Hkv = a.Hkv;
  p.Tq = a.Tq;
  p.Tk = a.Tk;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = reinterpret_cast<uint16_t*>(a.o);
  p.o_sb = a.o_sb;
  p.o_st = a.o_st;
  p.o_sh = a.o_sh;
  p.lse = a.lse;
  const int q_tiles = (a.Tq + ATT_BM - 1) / ATT_BM;
  p.n_pairs = (q_tiles + 1) / 2;
  p.total_items = a.B * a.H * p.n_pairs;
  p.status = status_word(device);
  const int grid = std::min(p.total_items, sm_count(device));
  const ItemList il = build_item_list(a, p.n_pairs, grid, device, stream);
  p.item_list = il.dev;
  p.items_per_cta = il.per_cta;
#ifdef RT_ATTN_PROF
  static long long* prof_buf = nullptr;
  if (!prof_buf) RT_CUDA_CHECK(cudaMallocManaged(&prof_buf, 148 * 2 * 8 * sizeof(long long)));
  p.prof = prof_buf;
  attn_prof_buffer() = prof_buf;
#endif
  kern<<<grid, ATT_PP_THREADS, S::TOTAL, stream>>>(tq, tk, tv, p);
  RT_LAUNCH_CHECK();
}

// Same contract as attn_fwd (flash_fwd.cu); requires scale > 0.
void attn_fwd_pp(const AttnArgs& a, cudaStream_t stream) {
  if (a.io_fp16) {
    if (a.D == 64) launch_fwd_pp<64, true, 8>(a, stream);
    else launch_fwd_pp<128, true, 8>(a, stream);
  } else if (a.D == 64) {
    launch_fwd_pp<64, false, 8>(a, stream);
  } else {
    launch_fwd_pp<128, false, 8>(a, stream);
  }
}

}  // namespace rt
