// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   TMA (plain per-CTA tiled loads, 128B swizzle) -> shared-memory ring
//   -> tcgen05.mma (one issuing thread, fp32 accumulators in TMEM, double buffered)
//   -> tcgen05.ld epilogue (bias / GELU / dGELU / residual / fp32 atomic accumulate).
//
//   C[b][m][n] = alpha * sum_k A[b][m][k] * B[b][n][k]   (+ epilogue)
//
// Each operand is either "K-major" (reduction dim contiguous: A stored [M][K], B stored
// [N][K]) or "MN-major" (A stored [K][M], B stored [K][N]).  That covers the three GEMMs of
// a Linear layer without any transposed copies:
//   forward  y  = x W^T      : A K-major (x),  B K-major (W[out][in])
//   dgrad    dx = dy W       : A K-major (dy), B MN-major (W as [K=out][N=in])
//   wgrad    dW = dy^T x     : A MN-major (dy as [K=tokens][M=out]), B MN-major (x)
// The reference's GPU matmul is a cuBLAS SGEMM wrapped in host<->device copies
// (src/gpu/cuda_enhanced.rs:122-159) plus naive/tiled scalar kernels
// (src/gpu/cuda_kernels.cu:59-75); this file replaces all of them.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (TMEM lane quarter = warp_id % 4; warps 2..5 take the left half of
// the tile's columns, warps 6..9 the right half).
//
// CTA-pair mode (template parameter PAIR): the kernel is launched as clusters of two CTAs that share one
// 256 x 256 tile through tcgen05.mma.cta_group::2.  Each CTA loads its 128 rows of A and its 128 rows of B
// (cp.async.bulk.tensor with .cta_group::2, no multicast: both halves complete on the even CTA's barrier), the even
// CTA's thread issues the MMAs for both, tcgen05.commit frees the stage in both CTAs, and each CTA's epilogue
// warps drain their own half of the accumulator.
#include <cstdlib>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;  // 2 control warps + 8 epilogue warps

struct GemmParams {
  int M, N, K, batch;
  void* C;
  long long ldc, c_batch_stride;
  const __nv_bfloat16* bias;  // [N] or null
  __nv_bfloat16* aux;         // same geometry as C (bf16) or null
  long long ld_aux, aux_batch_stride;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha (read by the epilogue warps)
  int epi_mode;
  int out_fp32;    // C is fp32 instead of bf16
  int accumulate;  // fp32 only: C += result using red.global.add.f32 (required when split_k > 1)
  int split_k;
  int m_blocks, n_blocks, k_blocks;
  int group;    // M-blocks per band of the tile order
  int c_tma, aux_tma;  // bf16 C / aux tiles leave through TMA stores (tensor maps tmap_c / tmap_aux are valid)
  int ab_fp16;  // A and B are fp16 instead of bf16 (C must then be fp32)
  int* status;
#ifdef RT_GEMM_PROF
  long long* prof;  // cycles the first worker's control threads spend in each wait (instrumented builds only)
#endif
};

#ifdef RT_GEMM_PROF
static long long* g_gemm_prof = nullptr;
extern "C" long long* rt_gemm_prof_buffer() { return g_gemm_prof; }
#define GPROF_T() clock64()
#define GPROF_ADD(slot, t0) do { if (worker == 0) acc_prof[slot] += clock64() - (t0); } while (0)
#else
#define GPROF_T() 0LL
#define GPROF_ADD(slot, t0) do { (void)(t0); } while (0)
#endif

// PAIR: two CTAs of a cluster work on one 256 x BLOCK_N tile with cta_group::2 MMAs; each CTA loads its 128 rows of A
// and its BLOCK_N / 2 rows of B, so a stage is a third smaller and the ring two stages deeper.
template <int BLOCK_N, bool PAIR = false>
struct GemmSmem {
  static constexpr int BN_LOAD = PAIR ? BLOCK_N / 2 : BLOCK_N;  // rows of B this CTA loads per stage
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BN_LOAD * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256 && !PAIR) ? 4 : 6;
  // epilogue staging: 8 warps x (32 rows x 128 B), 16-byte pieces XOR-swizzled by the row
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int EPI_BYTES = 8 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base, ctl
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static_assert(TOTAL <= 232448, "gemm: shared memory over the per-CTA limit");
};

__device__ __forceinline__ void decode_tile(int t, const GemmParams& p, int& split, int& b,
                                            int& mb, int& nb) {
  const int tiles_per_mat = p.m_blocks * p.n_blocks;
  const int per_batch = tiles_per_mat * p.split_k;
  b = t / per_batch;
  int r = t - b * per_batch;
  split = r / tiles_per_mat;
  r -= split * tiles_per_mat;
  // grouped ordering: M fastest inside bands of p.group M-blocks, so co-resident CTAs share A and B tiles through L2
  // and B is swept from DRAM once per band (the host picks the band height, see gemm_bf16)
  const int GROUP = p.group;
  const int band = GROUP * p.n_blocks;
  const int g = r / band;
  const int first_m = g * GROUP;
  const int rows = min(GROUP, p.m_blocks - first_m);
  const int in_band = r - g * band;
  mb = first_m + in_band % rows;
  nb = in_band / rows;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux,
                    const GemmParams p) {
  using S = GemmSmem<BLOCK_N, PAIR>;
  constexpr int STAGES = S::STAGES;
  // PAIR: launched as clusters of two CTAs.  p.m_blocks counts 256-row blocks; CTA `cta_rank` of the pair owns rows
  // [128 * cta_rank, 128 * cta_rank + 128) of A and of the accumulator and rows [BLOCK_N/2 * cta_rank, ...) of B.  The
  // even CTA issues every MMA; the odd CTA's TMA loads complete on the even CTA's barriers.
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int n_workers = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // 256 or 512, power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], PAIR ? 16 : 8);  // PAIR: the epilogue warps of both CTAs arrive on the even CTA's
    }
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_base_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // Programmatic dependent launch: the next kernel of the stream may start its prologue now (it becomes resident as
  // this grid's CTAs retire); this kernel's own first read of global memory and its first write wait for the
  // previous grid to complete (pdl_wait in the producer and epilogue roles; the MMA role touches no global memory).
  pdl_launch_dependents();

  const int total_tiles = p.batch * p.m_blocks * p.n_blocks * p.split_k;
  const int kb_per_split = (p.k_blocks + p.split_k - 1) / p.split_k;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
#ifdef RT_GEMM_PROF
      long long acc_prof[1] = {0};
#endif
      pdl_wait();
      for (int t = worker; t < total_tiles && ok; t += n_workers) {
        int split, b, mb, nb;
        decode_tile(t, p, split, b, mb, nb);
        if (PAIR) mb = mb * 2 + int(cta_rank);
        const int n_first = nb * BLOCK_N + int(cta_rank) * S::BN_LOAD;  // first row of B this CTA loads
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const long long tp0 = GPROF_T();
          if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          GPROF_ADD(0, tp0);
          uint8_t* sa = smem + s * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          if (PAIR) {
            // both CTAs' loads complete on the even CTA's barrier, which expects the bytes of both
            const uint32_t bar = mapa_shared(smem_u32(&full_bar[s]), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
            if (!A_MN) {
              tma_load_3d_pair(sa, &tmap_a, bar, kb * BLOCK_K, mb * BLOCK_M, b);
            } else {
#pragma unroll
              for (int c = 0; c < BLOCK_M / 64; ++c)
                tma_load_3d_pair(sa + c * 8192, &tmap_a, bar, mb * BLOCK_M + c * 64, kb * BLOCK_K, b);
            }
            if (!B_MN) {
              tma_load_3d_pair(sb, &tmap_b, bar, kb * BLOCK_K, n_first, b);
            } else {
#pragma unroll
              for (int c = 0; c < S::BN_LOAD / 64; ++c)
                tma_load_3d_pair(sb + c * 8192, &tmap_b, bar, n_first + c * 64, kb * BLOCK_K, b);
            }
            continue;
          }
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          if (!A_MN) {
            tma_load_3d(sa, &tmap_a, &full_bar[s], kb * BLOCK_K, mb * BLOCK_M, b);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_M / 64; ++c)
              tma_load_3d(sa + c * 8192, &tmap_a, &full_bar[s], mb * BLOCK_M + c * 64,
                          kb * BLOCK_K, b);
          }
          if (!B_MN) {
            tma_load_3d(sb, &tmap_b, &full_bar[s], kb * BLOCK_K, n_first, b);
          } else {
#pragma unroll
            for (int c = 0; c < S::BN_LOAD / 64; ++c)
              tma_load_3d(sb + c * 8192, &tmap_b, &full_bar[s], n_first + c * 64,
                          kb * BLOCK_K, b);
          }
        }
      }
#ifdef RT_GEMM_PROF
      if (worker == 0 && p.prof) p.prof[5 + cta_rank] = acc_prof[0];
#endif
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (PAIR && cta_rank != 0) {
      // odd CTA of a pair: its tiles are consumed by the even CTA's MMAs
    } else if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(PAIR ? 2 * BLOCK_M : BLOCK_M, BLOCK_N, A_MN, B_MN, !p.ab_fp16);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      bool ok = true;
#ifdef RT_GEMM_PROF
      long long acc_prof[5] = {0, 0, 0, 0, 0};
      const long long t_start = clock64();
#endif
      for (int t = worker; t < total_tiles && ok; t += n_workers, ++tile_i) {
        int split, b, mb, nb;
        decode_tile(t, p, split, b, mb, nb);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + kb_per_split);
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        const long long te0 = GPROF_T();
        if (!(PAIR ? mbar_wait_cluster(&tmem_empty[acc], acc_ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)
                   : mbar_wait(&tmem_empty[acc], acc_ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_MMA))) {
          ok = false;
          break;
        }
        GPROF_ADD(3, te0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const long long tf0 = GPROF_T();
          if (!mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          GPROF_ADD(1, tf0);
          const long long tq0 = GPROF_T();
          GPROF_ADD(2, tq0);
#ifdef RT_GEMM_PROF
          acc_prof[4] += 1;
#endif
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            if (PAIR) umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
            else umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) when these MMAs retire
          if (PAIR) {
            umma_commit_pair(smem_u32(&empty_bar[s]));
            umma_commit_pair(mapa_shared(smem_u32(&empty_bar[s]), 1));
          } else {
            umma_commit(&empty_bar[s]);
          }
        }
        if (ok) {
          if (PAIR) {
            umma_commit_pair(smem_u32(&tmem_full[acc]));
            umma_commit_pair(mapa_shared(smem_u32(&tmem_full[acc]), 1));
          } else {
            umma_commit(&tmem_full[acc]);
          }
        }
      }
#ifdef RT_GEMM_PROF
      if (worker == 0 && p.prof) {
        p.prof[0] = clock64() - t_start;
        for (int i = 1; i < 5; ++i) p.prof[i] = acc_prof[i];
      }
#endif
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_i = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 7) == 0) && (p.aux == nullptr || (p.ld_aux & 7) == 0);
    pdl_wait();
    const float alpha = p.alpha_dev ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
    for (int t = worker; t < total_tiles && ok; t += n_workers, ++tile_i) {
      int split, b, mb, nb;
      decode_tile(t, p, split, b, mb, nb);
      if (PAIR) mb = mb * 2 + int(cta_rank);
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int m = mb * BLOCK_M + row_in_tile;
      const bool row_ok = m < p.M;
      const bool add_bias = (p.bias != nullptr) && (split == 0);
      // bf16 outputs leave through shared memory when the 64-column pair is complete: a lane's 64 bytes of ITS row
      // become 128-byte row segments written by 8 lanes, so a store instruction touches 4 full lines instead of 32
      // half sectors (the per-lane path remains for fp32 / atomic outputs, ragged edges and unaligned rows)
      const bool staged_ok = !p.out_fp32 && vec_ok;
      uint8_t* wstage = smem + S::EPI_OFFSET + (warp - 2) * 4096;
      const int m_warp = mb * BLOCK_M + quarter * 32;  // first row of this warp
      auto stage_put = [&](int piece, uint4 w) {
        *reinterpret_cast<uint4*>(wstage + lane * 128 + ((piece ^ (lane & 7)) << 4)) = w;
      };
      // With a tensor map for the output the staged 32 x 64 tile leaves as ONE TMA store issued by lane 0 (the copy
      // engine writes whole lines and clips rows / columns beyond the matrix); the warp only waits, before it refills
      // the staging buffer, until the engine has read it.
      auto stage_flush = [&](const CUtensorMap* tm, int n_first, int bz) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m_warp < p.M) {
          tma_store_3d(tm, wstage, n_first, m_warp, bz);
          bulk_commit_group();
        }
      };
      auto stage_free = [&]() {
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
      };
      int n_store = 0;  // first column of the 64-column group being stored (read by the checked build only)
      auto stage_store = [&](__nv_bfloat16* base, long long ld) {  // base: row m_warp, column n0
        const int piece = lane & 7;
#pragma unroll
        for (int itr = 0; itr < 8; ++itr) {
          const int row = itr * 4 + (lane >> 3);
          if (m_warp + row < p.M) {
            const uint4 w = *reinterpret_cast<const uint4*>(wstage + row * 128 + ((piece ^ (row & 7)) << 4));
            // checked builds: the 8 columns this lane writes lie inside the row's N columns
            if (RT_GUARD(n_store + piece * 8 + 7, p.N, p.status))
              *reinterpret_cast<uint4*>(base + (long long)row * ld + piece * 8) = w;
          }
        }
      };
#pragma unroll 1
      for (int c = col_half * (BLOCK_N / 64); c < (col_half + 1) * (BLOCK_N / 64); c += 2) {
        const int n0 = nb * BLOCK_N + c * 32;
        if (n0 >= p.N) break;  // warp-uniform
        uint32_t r2[2][32];
        const uint32_t taddr = tmem_base + acc * BLOCK_N + c * 32 + (uint32_t(quarter * 32) << 16);
        __syncwarp();
        tmem_ld_32x32b_x32(taddr, r2[0]);
        tmem_ld_32x32b_x32(taddr + 32, r2[1]);
        tmem_ld_wait();
        if (staged_ok && n0 + 64 <= p.N) {
          n_store = n0;
          if (p.c_tma) stage_free();
          uint4 keep[2][4];  // GELU_DUAL: the bf16 pre-activations, reused for the second output
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int nh = n0 + h * 32;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r2[h][j]) * alpha;
            if (add_bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(p.bias[nh + j]);
            }
            if ((p.epi_mode == EPI_DGELU || p.epi_mode == EPI_RESIDUAL) && row_ok) {
              const uint4* src = reinterpret_cast<const uint4*>(p.aux + (long long)b * p.aux_batch_stride + (long long)m * p.ld_aux + nh);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 w = src[q];
                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = __bfloat1622float2(hh[e]);
                  if (p.epi_mode == EPI_DGELU) {
                    v[q * 8 + e * 2] *= gelu_tanh_grad(f.x);
                    v[q * 8 + e * 2 + 1] *= gelu_tanh_grad(f.y);
                  } else {
                    v[q * 8 + e * 2] += f.x;
                    v[q * 8 + e * 2 + 1] += f.y;
                  }
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              keep[h][q] = w;
              stage_put(h * 4 + q, w);
            }
          }
          __syncwarp();
          __nv_bfloat16* c_base = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)b * p.c_batch_stride + (long long)m_warp * p.ldc + n0;
          if (p.epi_mode == EPI_GELU_DUAL) {
            if (p.aux_tma) {
              stage_flush(&tmap_aux, n0, b);
              stage_free();
            } else {
              stage_store(p.aux + (long long)b * p.aux_batch_stride + (long long)m_warp * p.ld_aux + n0, p.ld_aux);
              __syncwarp();
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&keep[h][q]);
                float2 f0 = __bfloat1622float2(hh[0]), f1 = __bfloat1622float2(hh[1]);
                float2 f2 = __bfloat1622float2(hh[2]), f3 = __bfloat1622float2(hh[3]);
                uint4 w;
                w.x = pack_bf16x2(gelu_tanh(f0.x), gelu_tanh(f0.y));
                w.y = pack_bf16x2(gelu_tanh(f1.x), gelu_tanh(f1.y));
                w.z = pack_bf16x2(gelu_tanh(f2.x), gelu_tanh(f2.y));
                w.w = pack_bf16x2(gelu_tanh(f3.x), gelu_tanh(f3.y));
                stage_put(h * 4 + q, w);
              }
            __syncwarp();
          }
          if (p.c_tma) stage_flush(&tmap_c, n0, b);
          else stage_store(c_base, p.ldc);
          continue;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
        const int nq = n0 + h * 32;
        if (nq >= p.N) break;  // warp-uniform
        uint32_t(&r)[32] = r2[h];
        if (row_ok) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        const bool full_chunk = (nq + 32 <= p.N) && vec_ok;
        if (add_bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (nq + j < p.N) v[j] += __bfloat162float(p.bias[nq + j]);
        }
        __nv_bfloat16* aux_row =
            p.aux ? p.aux + (long long)b * p.aux_batch_stride + (long long)m * p.ld_aux + nq
                  : nullptr;
        if (p.epi_mode == EPI_GELU_DUAL) {
          if (full_chunk) {
            uint4* dst = reinterpret_cast<uint4*>(aux_row);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              dst[q] = w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + j < p.N) aux_row[j] = __float2bfloat16(v[j]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(__bfloat162float(__float2bfloat16(v[j])));
        } else if (p.epi_mode == EPI_DGELU || p.epi_mode == EPI_RESIDUAL) {
          float a[32];
          if (full_chunk) {
            const uint4* src = reinterpret_cast<const uint4*>(aux_row);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w = src[q];
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 f = __bfloat1622float2(h[e]);
                a[q * 8 + e * 2] = f.x;
                a[q * 8 + e * 2 + 1] = f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = (nq + j < p.N) ? __bfloat162float(aux_row[j]) : 0.f;
          }
          if (p.epi_mode == EPI_DGELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad(a[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += a[j];
          }
        }
        if (p.out_fp32) {
          float* crow = reinterpret_cast<float*>(p.C) + (long long)b * p.c_batch_stride +
                        (long long)m * p.ldc + nq;
          if (p.accumulate) {
            if (full_chunk) {
              float4* dst = reinterpret_cast<float4*>(crow);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                atomicAdd(dst + q, make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nq + j < p.N) atomicAdd(crow + j, v[j]);
            }
          } else if (full_chunk) {
            float4* dst = reinterpret_cast<float4*>(crow);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              dst[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + j < p.N) crow[j] = v[j];
          }
        } else {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) +
                                (long long)b * p.c_batch_stride + (long long)m * p.ldc + nq;
          if (full_chunk) {
            uint4* dst = reinterpret_cast<uint4*>(crow);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              dst[q] = w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + j < p.N) crow[j] = __float2bfloat16(v[j]);
          }
        }
        }  // row_ok
        }  // halves
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
        else mbar_arrive(&tmem_empty[acc]);
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // every TMA store of this warp has been performed
  }

  // Common exit: on abort give in-flight bulk copies time to land, then release TMEM.
  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA's shared or tensor memory goes away while the other may still touch it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool PAIR>
static void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
                        const GemmParams& p, int device, cudaStream_t stream) {
  using S = GemmSmem<BLOCK_N, PAIR>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, A_MN, B_MN, PAIR>;
  static int workers[64] = {0};  // persistent CTAs (or CTA pairs) that are resident at once on this device
  if (workers[device] == 0) {
    RT_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    int w = sm_count(device);
    if (PAIR) {
      // pairs cannot straddle the hardware's SM groups: ask how many fit at once
      cudaLaunchConfig_t probe{};
      probe.gridDim = dim3(unsigned(sm_count(device)) & ~1u);
      probe.blockDim = dim3(GEMM_THREADS);
      probe.dynamicSmemBytes = S::TOTAL;
      cudaLaunchAttribute at{};
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2;
      at.val.clusterDim.y = 1;
      at.val.clusterDim.z = 1;
      probe.attrs = &at;
      probe.numAttrs = 1;
      int clusters = 0;
      RT_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&clusters, kern, &probe));
      w = std::max(1, std::min(clusters, sm_count(device) / 2));
    }
    workers[device] = w;
  }
  const int total_tiles = p.batch * p.m_blocks * p.n_blocks * p.split_k;
  const int n_workers = std::min(total_tiles, workers[device]);
#ifdef RT_GEMM_PROF
  if (!g_gemm_prof) RT_CUDA_CHECK(cudaMallocManaged(&g_gemm_prof, 8 * sizeof(long long)));
  const_cast<GemmParams&>(p).prof = g_gemm_prof;
  g_gemm_prof[7] = n_workers;
#endif
  if (PAIR) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2u * unsigned(n_workers));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute at[2]{};
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 2;
    RT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, p));
    count_launch();
  } else {
    launch_pdl(kern, dim3(n_workers), dim3(GEMM_THREADS), S::TOTAL, stream, ta, tb, tc, tx, p);
    RT_LAUNCH_CHECK();
  }
}

void gemm_bf16(const GemmArgs& g, cudaStream_t stream) {
  if (g.M == 0 || g.N == 0 || g.batch == 0) return;
  RT_CHECK(g.K > 0, "gemm_bf16: empty reduction dimension");
  RT_CHECK(!g.accumulate || g.out_fp32, "gemm_bf16: accumulate needs an fp32 output");
  RT_CHECK(g.split_k >= 1, "gemm_bf16: split_k >= 1");
  RT_CHECK(g.split_k == 1 || g.accumulate, "gemm_bf16: split_k > 1 needs accumulate=true");
  RT_CHECK(g.epi_mode == EPI_NONE || g.aux != nullptr, "gemm_bf16: this epilogue needs aux");
  const int device = current_device();
  int block_n = (g.block_n == 128 || g.block_n == 256) ? g.block_n : 0;
  if (block_n == 0) block_n = (g.N <= 128) ? 128 : 256;
  // CTA pairs (one 256 x 256 tile per two SMs, a third less operand traffic from L2) measured level with single-CTA
  // tiles on the benchmarked shapes (+-5 % either way, run to run), and the training step does not move, so they are
  // opt-in: RUSTORCH_GEMM_PAIR=1 uses pairs wherever they are legal.
  const bool pair_legal = block_n == 256 && g.M > BLOCK_M;
  bool pair = false;
  if (const char* e = std::getenv("RUSTORCH_GEMM_PAIR")) pair = pair_legal && e[0] == '1';

  GemmParams p{};
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.batch = g.batch;
  p.C = g.c;
  p.ldc = g.ldc;
  p.c_batch_stride = g.c_batch_stride;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(g.bias);
  p.aux = reinterpret_cast<__nv_bfloat16*>(g.aux);
  p.ld_aux = g.ld_aux;
  p.aux_batch_stride = g.aux_batch_stride;
  p.alpha = g.alpha;
  p.alpha_dev = g.alpha_dev;
  p.epi_mode = g.epi_mode;
  p.out_fp32 = g.out_fp32;
  p.accumulate = g.accumulate;
  p.ab_fp16 = g.ab_fp16 ? 1 : 0;
  RT_CHECK(!g.ab_fp16 || (g.out_fp32 && !g.bias && !g.aux && g.epi_mode == EPI_NONE),
           "gemm: fp16 operands need an fp32 C and no fused epilogue");
  p.m_blocks = pair ? (g.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M) : (g.M + BLOCK_M - 1) / BLOCK_M;
  p.n_blocks = (g.N + block_n - 1) / block_n;
  p.k_blocks = (g.K + BLOCK_K - 1) / BLOCK_K;
  // Tile order: bands of `group` M-blocks, swept over all N-blocks.  B comes from DRAM once per band unless it stays in
  // L2 between bands, which a B larger than a fraction of L2 next to a streaming output does not (measured on
  // 16384 x 50304 x 768: 1.25 GB of DRAM reads for 102 MB of operands with bands of 8).  Then the band grows until
  // its rows of A are ~12 MB: fewer sweeps of B, and the band's A still lives in L2 through its sweep.
  {
    const double b_bytes = 2.0 * g.N * g.K, a_block_bytes = 2.0 * (pair ? 2 * BLOCK_M : BLOCK_M) * g.K;
    int group = 8;
    if (b_bytes > 24.0 * 1024 * 1024) group = std::max(8, std::min(64, int(12.0 * 1024 * 1024 / a_block_bytes)));
    p.group = std::min(group, std::max(1, p.m_blocks));
  }
  int sk = std::min(g.split_k, std::max(1, p.k_blocks));
  // every split must own at least one k-block
  while (sk > 1 && ((p.k_blocks + sk - 1) / sk) * (sk - 1) >= p.k_blocks) --sk;
  p.split_k = sk;
  p.status = status_word(device);

  const uint64_t M = g.M, N = g.N, K = g.K, B = g.batch;
  CUtensorMap ta = g.a_mn ? make_tmap_2byte(g.a, M, K, B, g.lda, g.a_batch_stride, 64, 64)
                          : make_tmap_2byte(g.a, K, M, B, g.lda, g.a_batch_stride, 64, BLOCK_M);
  CUtensorMap tb = g.b_mn ? make_tmap_2byte(g.b, N, K, B, g.ldb, g.b_batch_stride, 64, 64)
                          : make_tmap_2byte(g.b, K, N, B, g.ldb, g.b_batch_stride, 64, pair ? block_n / 2 : block_n);
  // Output tiles through TMA stores: bf16 C (and aux for the dual-output GELU epilogue) with 16-byte aligned base and
  // rows.  RUSTORCH_GEMM_TMA_STORE=0 keeps the per-lane stores.
  static const bool tma_store_on = [] {
    const char* e = std::getenv("RUSTORCH_GEMM_TMA_STORE");
    return !(e && e[0] == '0');
  }();
  auto storable = [&](const void* base, long long ld, long long bstride) {
    return tma_store_on && base != nullptr && (reinterpret_cast<uintptr_t>(base) & 15) == 0 && ld % 8 == 0 &&
           (g.batch == 1 || bstride % 8 == 0);
  };
  CUtensorMap tc = ta, tx = ta;
  if (!g.out_fp32 && storable(g.c, g.ldc, g.c_batch_stride)) {
    tc = make_tmap_2byte(g.c, N, M, B, g.ldc, g.c_batch_stride, 64, 32);
    p.c_tma = 1;
  }
  if (p.c_tma && g.epi_mode == EPI_GELU_DUAL && storable(g.aux, g.ld_aux, g.aux_batch_stride)) {
    tx = make_tmap_2byte(g.aux, N, M, B, g.ld_aux, g.aux_batch_stride, 64, 32);
    p.aux_tma = 1;
  }
#define RT_GEMM_DISPATCH(BN, PR)                                                              \
  if (!g.a_mn && !g.b_mn) launch_gemm<BN, false, false, PR>(ta, tb, tc, tx, p, device, stream);       \
  else if (!g.a_mn && g.b_mn) launch_gemm<BN, false, true, PR>(ta, tb, tc, tx, p, device, stream);    \
  else if (g.a_mn && g.b_mn) launch_gemm<BN, true, true, PR>(ta, tb, tc, tx, p, device, stream);      \
  else launch_gemm<BN, true, false, PR>(ta, tb, tc, tx, p, device, stream);
  if (pair) {
    RT_GEMM_DISPATCH(256, true)
  } else if (block_n == 256) {
    RT_GEMM_DISPATCH(256, false)
  } else {
    RT_GEMM_DISPATCH(128, false)
  }
#undef RT_GEMM_DISPATCH
}

}  // namespace rt
