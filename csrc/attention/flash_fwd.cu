// Flash-attention forward on tcgen05 (sm_100a): causal / non-causal, MHA and GQA, head
// dim 64 or 128, bf16 in, fp32 softmax statistics, bf16 out + fp32 log-sum-exp.
//
// One CTA = one 128-row query tile of one (batch, head).  Warps 0..3 (128 threads) each own
// one score row; warp 4 lane 0 issues every TMA load and every tcgen05.mma:
//   S  = Q K_j^T          -> TMEM columns [0,128)
//   row threads: online softmax on S (two TMEM passes, 32 columns at a time), P (bf16) into the
//                swizzled staging tile in shared memory
//   Ob = P V_j            -> TMEM columns [128,128+D)   (fresh each block)
//   row threads: O = O * exp2(m_old - m_new) + Ob    (fp32 in registers)
// K/V tiles stream through a 2-deep TMA ring.  The score matrix never reaches HBM, unlike
// the reference, which materialises [B,H,T,T] scores (src/nn/transformer_phase6.rs:342-374)
// and whose "fused_attention" kernel string is never compiled (src/gpu/custom_kernels.rs:439-536).
#include "../api.h"
#include "../common/launch.h"
#include "attn_common.cuh"

namespace rt {

struct AttnFwdParams {
  int B, H, Hkv, Tq, Tk;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* o;
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
  // q_full, kv_full[2], kv_empty[2], s_full, p_full, o_full
  static constexpr int TOTAL = OFF_BAR + 8 * 8 + 16;
};

template <int D>
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
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
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
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
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
      constexpr uint32_t idesc_S = make_idesc_f16(128, 128, false, false, true);
      constexpr uint32_t idesc_PV = make_idesc_f16(128, D, false, true, true);
      bool ok = true;
      mbar_arrive_expect_tx(q_full, S::TILE);
      load_tile<D>(sQ, &tmap_q, q_full, q0, h, b);
      mbar_arrive_expect_tx(&kv_full[0], 2 * S::TILE);
      load_tile<D>(smem + S::OFF_K, &tmap_k, &kv_full[0], 0, hk, b);
      load_tile<D>(smem + S::OFF_V, &tmap_v, &kv_full[0], 0, hk, b);
      ok = mbar_wait(q_full, 0, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) {
          const int s2 = (j + 1) & 1;
          if (!mbar_wait(&kv_empty[s2], (((j + 1) >> 1) & 1) ^ 1, ctl, p.status,
                         RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[s2], 2 * S::TILE);
          load_tile<D>(smem + S::OFF_K + s2 * S::TILE, &tmap_k, &kv_full[s2], (j + 1) * ATT_BN, hk,
                       b);
          load_tile<D>(smem + S::OFF_V + s2 * S::TILE, &tmap_v, &kv_full[s2], (j + 1) * ATT_BN, hk,
                       b);
        }
        if (!mbar_wait(&kv_full[s], (j >> 1) & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ);
        const uint32_t aK = smem_u32(smem + S::OFF_K + s * S::TILE);
        const uint32_t aV = smem_u32(smem + S::OFF_V + s * S::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem_S, tile_desc_kmajor<D>(aQ, kk), tile_desc_kmajor<D>(aK, kk), idesc_S,
                      kk > 0 ? 1u : 0u);
        umma_commit(s_full);
        if (!mbar_wait(p_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t aP = smem_u32(sP);
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          umma_f16_ss(tmem_O, stage_desc_kmajor(aP, kk), tile_desc_mnmajor<D>(aV, kk), idesc_PV,
                      kk > 0 ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_sel = uint32_t(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int col_base = j * ATT_BN;
      const int limit = p.causal ? min(p.Tk - 1, qi + off) : (p.Tk - 1);  // last visible column
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_S + lane_sel + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]) * p.scale_log2;
          if (col_base + c * 32 + i <= limit) mx = fmaxf(mx, s);
        }
      }
      const float m_new = mx;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_S + lane_sel + c * 32, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]) * p.scale_log2;
          const float e = (col_base + c * 32 + i <= limit) ? exp2f(s - m_use) : 0.f;
          pv[i] = e;
          rowsum += e;
        }
        stage_row_chunk_bf16(sP, row, c * 32, pv);
      }
      l = l * alpha + rowsum;
      m = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
      if (!mbar_wait(o_full, j & 1, ctl, p.status, RT_ERR_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_O + lane_sel + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
    }
    if (ok && qi < p.Tq) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.o + (long long)b * p.o_sb + (long long)qi * p.o_st + (long long)h * p.o_sh;
#pragma unroll
      for (int q = 0; q < D / 8; ++q) {
        uint4 w;
        w.x = pack_bf16x2(o_acc[q * 8 + 0] * inv, o_acc[q * 8 + 1] * inv);
        w.y = pack_bf16x2(o_acc[q * 8 + 2] * inv, o_acc[q * 8 + 3] * inv);
        w.z = pack_bf16x2(o_acc[q * 8 + 4] * inv, o_acc[q * 8 + 5] * inv);
        w.w = pack_bf16x2(o_acc[q * 8 + 6] * inv, o_acc[q * 8 + 7] * inv);
        reinterpret_cast<uint4*>(orow)[q] = w;
      }
      p.lse[((long long)b * p.H + h) * p.Tq + qi] =
          l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
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

template <int D>
static void launch_fwd(const AttnArgs& a, cudaStream_t stream) {
  using S = AttnFwdSmem<D>;
  const int device = current_device();
  auto kern = attn_fwd_kernel<D>;
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
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
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
  if (a.D == 64) launch_fwd<64>(a, stream);
  else launch_fwd<128>(a, stream);
}

}  // namespace rt
