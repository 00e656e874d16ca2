// Flash-attention forward on tcgen05 (sm_100a): causal / non-causal, MHA and GQA, head
// dim 64 or 128, bf16 in, fp32 softmax statistics, bf16 out + fp32 log-sum-exp.
//
// One CTA = one 128-row query tile of one (batch, head).  Warps 0..3 (128 threads) each own
// one score row; warp 4 lane 0 issues every TMA load and every tcgen05.mma:
//   S  = Q K_j^T          -> TMEM columns [0,128)
//   row threads: pull their whole S row into registers (one wait), release S at once so the
//                MMA of the NEXT key tile overlaps this tile's softmax, exponentiate against a
//                running reference maximum and stage P (bf16) in shared memory
//   O += P V_j            -> TMEM columns [128,128+D), accumulated by the tensor core
// The reference maximum is only raised (and O / l rescaled through a TMEM load-scale-store)
// when a row's block maximum exceeds it by more than 2^8; until then exponentials are taken
// against the stale maximum, which the final division by l cancels exactly.  K and V tiles
// stream through separate 2-deep TMA rings (K is released as soon as its S MMA retires).
// The score matrix never reaches HBM, unlike the reference, which materialises [B,H,T,T]
// scores (src/nn/transformer_phase6.rs:342-374) and whose "fused_attention" kernel string is
// never compiled (src/gpu/custom_kernels.rs:439-536).
#include "../api.h"
#include "../common/launch.h"
#include "attn_common.cuh"

#include <cstdlib>
#include <string>

namespace rt {

void attn_fwd_pp(const AttnArgs& a, cudaStream_t stream);  // flash_fwd_pp.cu

struct AttnFwdParams {
  int B, H, Hkv, Tq, Tk;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  uint16_t* o;   // bf16, or fp16 in the F16 instantiation
  long long o_sb, o_st, o_sh;
  float* lse;  // [B][H][Tq]
  int* status;
};

template <int D>
struct AttnFwdSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE;
  static constexpr int OFF_V = 3 * TILE;
  static constexpr int OFF_P = 5 * TILE;
  static constexpr int OFF_BAR = OFF_P + 2 * ATT_HALF_BYTES;
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_empty, p_full, pv_done
  static constexpr int TOTAL = OFF_BAR + 13 * 8 + 16;
};

constexpr float ATT_RESCALE_THRESHOLD = 8.f;  // log2 units

// F16: q / k / v / o are fp16 (the quantised LLM runtime's activations); P is then staged as fp16 too.
template <int D, bool F16>
__global__ void __launch_bounds__(160, (D == 64) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnFwdParams p) {
  using S = AttnFwdSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint8_t* sQ = smem + S::OFF_Q;
  uint8_t* sP = smem + S::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* s_empty = bars + 10;
  uint64_t* p_full = bars + 11;
  uint64_t* pv_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * ATT_BM;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  constexpr uint32_t TMEM_COLS = 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;

  const int off = p.Tk - p.Tq;  // causal: key col visible iff col <= row + off
  int n_kv = (p.Tk + ATT_BN - 1) / ATT_BN;
  if (p.causal) {
    const int last_col = min(p.Tk - 1, q0 + ATT_BM - 1 + off);
    n_kv = last_col < 0 ? 0 : min(n_kv, last_col / ATT_BN + 1);
  }

  if (warp == 4) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, !F16);
      constexpr uint32_t idesc_PV = make_idesc_f16(128, D, false, true, !F16);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      auto kbuf = [&](int s) { return smem + S::OFF_K + s * S::TILE; };
      auto vbuf = [&](int s) { return smem + S::OFF_V + s * S::TILE; };
      auto issue_S = [&](int s) {
        const uint32_t aK = smem_u32(kbuf(s));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S, kk > 0 ? 1u : 0u);
        umma_commit(s_full);
        umma_commit(&k_empty[s]);
      };
      bool ok = true;
      mbar_arrive_expect_tx(q_full, S::TILE);
      load_tile<D>(sQ, &tmap_q, q_full, q0, h, b);
      for (int j = 0; j < min(2, n_kv); ++j) {
        mbar_arrive_expect_tx(&k_full[j], S::TILE);
        load_tile<D>(kbuf(j), &tmap_k, &k_full[j], j * ATT_BN, hk, b);
        mbar_arrive_expect_tx(&v_full[j], S::TILE);
        load_tile<D>(vbuf(j), &tmap_v, &v_full[j], j * ATT_BN, hk, b);
      }
      ok = mbar_wait(q_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER) &&
           mbar_wait(&k_full[0], 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      if (ok) {
        tc_fence_after();
        issue_S(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_kv) {  // S of the next key tile as soon as the row threads hold S(j) in registers
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&k_full[s1], ((j + 1) >> 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) &&
               mbar_wait(s_empty, j & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_S(s1);
        }
        if (j + 2 < n_kv) {  // refill this K stage once S(j) has retired
          if (!mbar_wait(&k_empty[s], ph, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[s], S::TILE);
          load_tile<D>(kbuf(s), &tmap_k, &k_full[s], (j + 2) * ATT_BN, hk, b);
        }
        ok = mbar_wait(&v_full[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA) &&
             mbar_wait(p_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(vbuf(s));
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          umma_f16_ss(tmem_O, stage_desc_kmajor(aP, kk), tile_desc_mnmajor<D>(aV, kk), idesc_PV,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(pv_done);
        umma_commit(&v_empty[s]);
        if (j + 2 < n_kv) {  // refill this V stage once PV(j) has retired
          if (!mbar_wait(&v_empty[s], ph, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[s], S::TILE);
          load_tile<D>(vbuf(s), &tmap_v, &v_full[s], (j + 2) * ATT_BN, hk, b);
        }
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_sel = uint32_t(warp * 32) << 16;
    const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);  // last visible column
    float m = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[128];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld_32x32b_x32(tmem_S + lane_sel + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_empty);  // S is in registers: the next S MMA may overwrite TMEM now
      const int col_base = j * ATT_BN;
      // masking is only needed on the tile that crosses the causal diagonal or the end of the keys
      const bool partial = (col_base + ATT_BN - 1 > q0 + off && p.causal) || (col_base + ATT_BN > p.Tk);
      float mx = -INFINITY;
      if (partial) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float s = __uint_as_float(r[i]) * p.scale_log2;
          s = (col_base + i <= limit) ? s : -INFINITY;
          r[i] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const float s = __uint_as_float(r[i]) * p.scale_log2;
          r[i] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      }
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m = (mx == -INFINITY) ? 0.f : mx;
      } else {
        rescale = __any_sync(0xffffffffu, mx > m + ATT_RESCALE_THRESHOLD);
        if (rescale) {
          const float m_new = fmaxf(m, mx);
          alpha = ex2_approx(m - m_new);
          m = m_new;
          l *= alpha;
        }
      }
      float rowsum = 0.f;
#pragma unroll
      for (int i = 0; i < 128; ++i) {
        const float e = ex2_approx(__uint_as_float(r[i]) - m);
        r[i] = __float_as_uint(e);
        rowsum += e;
      }
      l += rowsum;
      // P(j-1) V(j-1) must have retired before the staging tile is overwritten or O is rescaled
      if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) { ok = false; break; }
      if (rescale) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          __syncwarp();
          tmem_ld_32x32b_x32(tmem_O + lane_sel + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x32(tmem_O + lane_sel + c * 32, o);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[i] = __uint_as_float(r[c * 32 + i]);
        stage_row_chunk_bf16<F16>(sP, row, c * 32, pv);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && n_kv > 0) ok = mbar_wait(pv_done, (n_kv - 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE);
    tc_fence_after();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    uint16_t* orow = p.o + (long long)b * p.o_sb + (long long)qi * p.o_st + (long long)h * p.o_sh;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      if (ok && n_kv > 0) {
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_O + lane_sel + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (ok && qi < p.Tq) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_2x16<F16>(__uint_as_float(o[q * 8 + 0]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
          w.y = pack_2x16<F16>(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
          w.z = pack_2x16<F16>(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
          w.w = pack_2x16<F16>(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
          reinterpret_cast<uint4*>(orow + c * 32)[q] = w;
        }
      }
    }
    if (ok && qi < p.Tq)
      p.lse[((long long)b * p.H + h) * p.Tq + qi] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    tc_fence_before();
  }

  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, bool F16>
static void launch_fwd(const AttnArgs& a, cudaStream_t stream) {
  using S = AttnFwdSmem<D>;
  const int device = current_device();
  auto kern = attn_fwd_kernel<D, F16>;
  static bool configured[64] = {false};
  if (!configured[device]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device] = true;
  }
  CUtensorMap tq = make_tmap_2byte_4d(a.q, D, a.Tq, a.H, a.B, a.q_st, a.q_sh, a.q_sb, 64, 128);
  CUtensorMap tk = make_tmap_2byte_4d(a.k, D, a.Tk, a.Hkv, a.B, a.k_st, a.k_sh, a.k_sb, 64, 128);
  CUtensorMap tv = make_tmap_2byte_4d(a.v, D, a.Tk, a.Hkv, a.B, a.v_st, a.v_sh, a.v_sb, 64, 128);
  AttnFwdParams p{};
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
  p.status = status_word(device);
  dim3 grid((a.Tq + ATT_BM - 1) / ATT_BM, a.H, a.B);
  kern<<<grid, 160, S::TOTAL, stream>>>(tq, tk, tv, p);
  RT_LAUNCH_CHECK();
}

void attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  RT_CHECK(a.D == 64 || a.D == 128, "attention: head_dim must be 64 or 128");
  RT_CHECK(a.H % a.Hkv == 0, "attention: n_heads must be a multiple of n_kv_heads");
  RT_CHECK((a.o_st % 8) == 0 && (a.o_sh % 8) == 0 && (a.o_sb % 8) == 0,
           "attention: output strides must be multiples of 8 elements");
  if (a.B == 0 || a.Tq == 0) return;
  // Default: the persistent ping-pong kernel (flash_fwd_pp.cu).  RUSTORCH_ATTN_FWD=tile selects the one-CTA-per-query-tile
  // kernel of this file, which is also used for a non-positive softmax scale.
  static const bool use_tile_kernel = [] {
    const char* e = std::getenv("RUSTORCH_ATTN_FWD");
    return e != nullptr && std::string(e) == "tile";
  }();
  if (!use_tile_kernel && a.scale > 0.f) {
    attn_fwd_pp(a, stream);
    return;
  }
  if (a.io_fp16) {
    if (a.D == 64) launch_fwd<64, true>(a, stream);
    else launch_fwd<128, true>(a, stream);
  } else if (a.D == 64) {
    launch_fwd<64, false>(a, stream);
  } else {
    launch_fwd<128, false>(a, stream);
  }
}

}  // namespace rt
