// Tensor-parallel linear layers as ONE kernel each: the collective runs inside the GEMM, tile by tile,
// over NVLink peer memory (symmetric allocations), instead of NCCL before / after a library GEMM.
//
//   MODE_AG (all-gather -> GEMM, column-parallel forward / row-parallel dgrad)
//     y[M][N] = concat_r(x_r)[M][K] . B^T          x_r: every rank's [M/W][K] shard in symmetric memory
//     A few "copy CTAs" stream the remote shards into a local gather buffer with the bulk-copy engine
//     (cp.async.bulk global -> shared -> global, a ring of 32-48 KB pieces driven by one thread, several
//     hundred KB in flight per CTA, so 8 CTAs keep an NVLink port busy) and publish one flag per 128-row
//     block.  The compute CTAs run the tcgen05 GEMM over the local shard first and then over the remote
//     blocks in arrival order; their TMA producer waits on the block's flag, so math on block i overlaps the
//     transfer of blocks > i.  Every remote byte crosses NVLink exactly once (peer reads are not cached in
//     the reader's L2, so loading A tiles straight from the peer would cross once per N-block).
//
//   MODE_RS (GEMM -> reduce-scatter, row-parallel forward / column-parallel dgrad)
//     out_r[M/W][N] = sum_src (x_src . B_src^T)[rows of r]
//     Tiles for remote owners are computed first: the epilogue turns each warp's 32 x 64 piece of the tile
//     into row-major bf16 in shared memory and stores it to the OWNER rank's staging buffer over NVLink as
//     128-byte row segments, then bumps a per-(block, source) counter there, so the transfer overlaps the
//     remaining math.  The rank's own rows come last and never leave the chip as partials: their epilogue
//     waits for the W-1 sources' counters of the block, adds the staged partials (+ bias, + residual) to the
//     fp32 accumulator straight out of TMEM and writes the bf16 result.  No separate reduce phase.  Staging
//     is double-buffered by call parity, which makes reuse safe without a second barrier (a rank can never
//     be two calls ahead of a peer, because each call's own-row tiles need that peer's partials of the same
//     call).
//
// Synchronisation is by flags in symmetric memory (st.release.sys / red.release.sys / ld.acquire.sys),
// every wait is bounded by a globaltimer deadline and reports through the status word; on a timeout the
// CTA drains its copies, frees TMEM and leaves.  All CTAs of a launch are co-resident (grid <= SM count,
// one CTA per SM), so waits inside one launch cannot dead-lock on scheduling.  No multicast anywhere.
//
// The reference has no tensor-parallel compute path: its ColumnParallel/RowParallel "layers" slice a weight
// on the host and call a blocking all-reduce stub (src/distributed/model_parallel.rs:429-503).
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

constexpr int TP_BLOCK_M = 128;
constexpr int TP_BLOCK_K = 64;
constexpr int TP_UMMA_K = 16;
constexpr int TP_THREADS = 320;

struct TpParams {
  int mode;  // 0 = AG, 1 = RS
  int M, N, K;
  int m_blocks, n_blocks, k_blocks, mbs;  // mbs = 128-row blocks per shard
  int world, rank, epoch, n_comm;
  unsigned long long timeout_ns;
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ld_res;
  // AG
  const __nv_bfloat16* x_peer[RT_MAX_PEERS];
  __nv_bfloat16* xg;
  int* mb_ready;        // local, [m_blocks], holds the epoch of the last completed fetch
  unsigned* comm_done;  // local counter
  // RS
  __nv_bfloat16* stage_peer[RT_MAX_PEERS];
  long long stage_parity_stride;  // elements between the two parities
  // flags (symmetric): [0,W) shard_ready, [W,2W) pull_done, [2W, 2W + mbs*W) rs_count[mbl][src]
  int* flags_peer[RT_MAX_PEERS];
  int* status;
};

template <int BLOCK_N>
struct TpSmem {
  static constexpr int A_BYTES = TP_BLOCK_M * TP_BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * TP_BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;  // 8 epilogue warps x (32 rows x 128 B), 16-byte pieces XOR-swizzled
  static constexpr int EPI_BYTES = 8 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static_assert(TOTAL <= 232448, "tp_gemm: shared memory over the per-CTA limit");
};

__device__ __forceinline__ void tp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void tp_st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int tp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int tp_ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void tp_fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ uint4 tp_ld_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Spin until *p >= want (acquire, system or gpu scope); false on timeout / CTA abort.
template <bool SYS>
__device__ __forceinline__ bool tp_wait_ge(const int* p, int want, const TpParams& P, CtaCtl* ctl) {
  if ((SYS ? tp_ld_acquire_sys(p) : tp_ld_acquire_gpu(p)) >= want) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned it = 0;
  while ((SYS ? tp_ld_acquire_sys(p) : tp_ld_acquire_gpu(p)) < want) {
    if ((++it & 0xff) == 0) {
      if (ctl && ctl->abort) return false;
      if (globaltimer_ns() - t0 > P.timeout_ns) {
        if (ctl) ctl->abort = 1;
        atomicCAS(P.status, 0, RT_ERR_TIMEOUT_PEER);
        return false;
      }
    }
    __nanosleep(40);
  }
  return true;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Processing order -> global 128-row block.  AG: own shard first, then the peers in ring order (the
// order the copy CTAs fetch them).  RS: peers' rows first (their tiles travel while the rest is computed),
// own rows last.
__device__ __forceinline__ int tp_block_at(int pm, const TpParams& P) {
  const int s = pm / P.mbs, j = pm - s * P.mbs;
  const int shard = P.mode == 0 ? (P.rank + s) % P.world : (P.rank + 1 + s) % P.world;
  return shard * P.mbs + j;
}

__device__ __forceinline__ void tp_decode(int t, const TpParams& P, int& gmb, int& nb) {
  constexpr int GROUP = 8;
  const int band = GROUP * P.n_blocks;
  const int g = t / band;
  const int first = g * GROUP;
  const int rows = min(GROUP, P.m_blocks - first);
  const int in_band = t - g * band;
  gmb = tp_block_at(first + in_band % rows, P);
  nb = in_band / rows;
}

template <int BLOCK_N, bool B_MN>
__global__ void __launch_bounds__(TP_THREADS, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,   // AG: local shard [Ms][K]; RS: x [M][K]
               const __grid_constant__ CUtensorMap tmap_ag,  // AG: gather buffer [M][K]; RS: unused copy of tmap_a
               const __grid_constant__ CUtensorMap tmap_b, const TpParams P) {
  using S = TpSmem<BLOCK_N>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(P.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = P.world, R = P.rank;
  const bool is_comm = P.mode == 0 && (int)blockIdx.x < P.n_comm;
  int* my_flags = P.flags_peer[R];

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_ag);
    tma_prefetch_desc(&tmap_b);
  }
  __syncthreads();

  if (is_comm) {
    // ======================================================================= copy CTA (AG mode)
    if (threadIdx.x == 0) {
      bool ok = true;
      if (blockIdx.x == 0) {  // this rank's shard is final (earlier kernels on the stream wrote it): tell the peers
        __threadfence_system();
        for (int p = 0; p < W; ++p)
          if (p != R) tp_st_release_sys(P.flags_peer[p] + R, P.epoch);
      }
      const long long blk_bytes = (long long)TP_BLOCK_M * P.K * 2;
      constexpr uint32_t PIECE = S::STAGE_BYTES;
      uint32_t cnt = 0;  // pieces issued so far (ring position)
      int unit = 0;
      for (int s = 1; s <= W && ok; ++s) {
        const int src = (R + s) % W;  // peers in ring order, own shard last
        if (src != R) ok = tp_wait_ge<true>(my_flags + src, P.epoch, P, ctl);
        for (int j = 0; j < P.mbs && ok; ++j, ++unit) {
          if (unit % P.n_comm != (int)blockIdx.x) continue;
          const uint8_t* gsrc = reinterpret_cast<const uint8_t*>(P.x_peer[src]) + (long long)j * blk_bytes;
          const int gmb = src * P.mbs + j;
          uint8_t* gdst = reinterpret_cast<uint8_t*>(P.xg) + (long long)gmb * blk_bytes;
          const int pieces = (int)((blk_bytes + PIECE - 1) / PIECE);
          auto piece_bytes = [&](int q) { return (uint32_t)min((long long)PIECE, blk_bytes - (long long)q * PIECE); };
          // prologue: fill the ring
          const uint32_t base = cnt;
          for (int q = 0; q < pieces && q < STAGES; ++q) {
            const uint32_t st = (base + q) % STAGES;
            mbar_arrive_expect_tx(&full_bar[st], piece_bytes(q));
            bulk_g2s(smem + st * PIECE, gsrc + (long long)q * PIECE, piece_bytes(q), &full_bar[st]);
          }
          for (int q = 0; q < pieces && ok; ++q) {
            const uint32_t c = base + q, st = c % STAGES, ph = (c / STAGES) & 1;
            ok = mbar_wait(&full_bar[st], ph, ctl, P.status, RT_ERR_TIMEOUT_PEER);
            if (!ok) break;
            bulk_s2g(gdst + (long long)q * PIECE, smem + st * PIECE, piece_bytes(q));
            bulk_commit();
            // refill the stage whose store was committed one step ago (it has been read by now or soon)
            if (q >= 1 && q - 1 + STAGES < pieces) {
              bulk_wait_read<1>();
              const int nq = q - 1 + STAGES;
              const uint32_t nst = (base + nq) % STAGES;
              mbar_arrive_expect_tx(&full_bar[nst], piece_bytes(nq));
              bulk_g2s(smem + nst * PIECE, gsrc + (long long)nq * PIECE, piece_bytes(nq), &full_bar[nst]);
            }
          }
          bulk_wait_all();  // stores have landed (also drains the ring before the next unit reuses it)
          cnt = base + pieces;
          if (ok) {
            tp_fence_proxy_async_all();
            __threadfence();
            tp_st_release_gpu(P.mb_ready + gmb, P.epoch);
          }
        }
      }
      // last copy CTA to finish tells the peers that this rank no longer reads their shards, then
      // copy CTA 0 keeps the kernel alive until every peer has said the same about this rank's shard.
      __threadfence();
      const unsigned done = atomicAdd(P.comm_done, 1u) + 1;
      if (ok && done == (unsigned)P.n_comm * (unsigned)P.epoch) {
        for (int p = 0; p < W; ++p)
          if (p != R) tp_st_release_sys(P.flags_peer[p] + W + R, P.epoch);
      }
      if (blockIdx.x == 0) {
        for (int p = 0; p < W && ok; ++p)
          if (p != R) ok = tp_wait_ge<true>(my_flags + W + p, P.epoch, P, ctl);
      }
    }
    __syncthreads();
    return;
  }

  // =========================================================================== compute CTA
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  const int cta = (int)blockIdx.x - (P.mode == 0 ? P.n_comm : 0);
  const int n_cta = (int)gridDim.x - (P.mode == 0 ? P.n_comm : 0);
  const int total_tiles = P.m_blocks * P.n_blocks;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int waited_mb = -1;
      for (int t = cta; t < total_tiles && ok; t += n_cta) {
        int gmb, nb;
        tp_decode(t, P, gmb, nb);
        const bool local_rows = P.mode == 0 && gmb / P.mbs == R;
        if (P.mode == 0 && !local_rows && waited_mb != gmb) {
          ok = tp_wait_ge<false>(P.mb_ready + gmb, P.epoch, P, ctl);
          if (!ok) break;
          tp_fence_proxy_async_all();  // the block was written through the async proxy by a copy CTA
          waited_mb = gmb;
        }
        const CUtensorMap* ta = (P.mode == 0 && !local_rows) ? &tmap_ag : &tmap_a;
        const int arow = (P.mode == 0 && local_rows) ? (gmb - R * P.mbs) * TP_BLOCK_M : gmb * TP_BLOCK_M;
        for (int kb = 0; kb < P.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, P.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_3d(sa, ta, &full_bar[s], kb * TP_BLOCK_K, arow, 0);
          if (!B_MN) {
            tma_load_3d(sb, &tmap_b, &full_bar[s], kb * TP_BLOCK_K, nb * BLOCK_N, 0);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c)
              tma_load_3d(sb + c * 8192, &tmap_b, &full_bar[s], nb * BLOCK_N + c * 64, kb * TP_BLOCK_K, 0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(TP_BLOCK_M, BLOCK_N, false, B_MN, true);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_cta, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, ctl, P.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < P.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, ctl, P.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TP_BLOCK_K / TP_UMMA_K; ++kk) {
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * (TP_UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (TP_UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sb + kk * (TP_UMMA_K * 2), 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_i = 0;
    bool ok = true;
    const long long Ms = (long long)P.mbs * TP_BLOCK_M;
    for (int t = cta; t < total_tiles && ok; t += n_cta, ++tile_i) {
      int gmb, nb;
      tp_decode(t, P, gmb, nb);
      const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, ctl, P.status, RT_ERR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      __nv_bfloat16* row_ptr;
      int dst = R, mbl = 0;
      const __nv_bfloat16* part = nullptr;  // RS, own rows: the sources' staged partials of this row
      if (P.mode == 0) {
        row_ptr = P.C + ((long long)gmb * TP_BLOCK_M + row_in_tile) * P.ldc;
      } else {
        dst = gmb / P.mbs;
        mbl = gmb - dst * P.mbs;
        const long long parity_off = (long long)(P.epoch & 1) * P.stage_parity_stride;
        if (dst == R) {
          // own rows: every other source has sent all its tiles of this 128-row block?
          const int want = P.epoch * 8 * P.n_blocks;  // 8 epilogue warps signal once per tile
          bool arrived = true;
          if (lane < W && lane != R) arrived = tp_wait_ge<true>(my_flags + 2 * W + mbl * W + lane, want, P, ctl);
          if (!__all_sync(0xffffffffu, arrived)) {
            ok = false;
            break;
          }
          row_ptr = P.C + ((long long)mbl * TP_BLOCK_M + row_in_tile) * P.ldc;
          part = P.stage_peer[R] + parity_off + ((long long)mbl * TP_BLOCK_M + row_in_tile) * P.N;
        } else {
          // staging of the owner: [parity][src = R][Ms][N]; row_ptr = first row of this warp's 32
          row_ptr = P.stage_peer[dst] + parity_off + ((long long)R * Ms + (long long)mbl * TP_BLOCK_M + quarter * 32) * P.N;
        }
      }
      const bool remote = P.mode == 1 && dst != R;
      uint8_t* wstage = smem + S::EPI_OFFSET + (warp - 2) * 4096;
#pragma unroll 1
      for (int c = col_half * (BLOCK_N / 64); c < (col_half + 1) * (BLOCK_N / 64); c += 2) {
        const int n0 = nb * BLOCK_N + c * 32;
        if (n0 >= P.N) break;
        const bool full = n0 + 64 <= P.N;
        uint32_t r[2][32];
        const uint32_t taddr = tmem_base + acc * BLOCK_N + c * 32 + (uint32_t(quarter * 32) << 16);
        __syncwarp();
        tmem_ld_32x32b_x32(taddr, r[0]);
        tmem_ld_32x32b_x32(taddr + 32, r[1]);
        tmem_ld_wait();
        if (remote && full) {
          // row-major through shared memory: lane = row writes its eight 16-byte pieces, then eight lanes
          // cover one row's 128 bytes, so every store instruction sends four full 128-byte segments
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int hq = q >> 2, o = (q & 3) * 8;
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[hq][o + 0]), __uint_as_float(r[hq][o + 1]));
            w.y = pack_bf16x2(__uint_as_float(r[hq][o + 2]), __uint_as_float(r[hq][o + 3]));
            w.z = pack_bf16x2(__uint_as_float(r[hq][o + 4]), __uint_as_float(r[hq][o + 5]));
            w.w = pack_bf16x2(__uint_as_float(r[hq][o + 6]), __uint_as_float(r[hq][o + 7]));
            *reinterpret_cast<uint4*>(wstage + lane * 128 + ((q ^ (lane & 7)) << 4)) = w;
          }
          __syncwarp();
          const int piece = lane & 7;
#pragma unroll
          for (int itr = 0; itr < 8; ++itr) {
            const int row = itr * 4 + (lane >> 3);
            const uint4 w = *reinterpret_cast<const uint4*>(wstage + row * 128 + ((piece ^ (row & 7)) << 4));
            *reinterpret_cast<uint4*>(row_ptr + (long long)row * P.N + n0 + piece * 8) = w;
          }
          continue;
        }
        // direct path: this lane's row, 32 columns at a time
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int nh = n0 + h * 32;
          if (nh >= P.N) break;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[h][j]);
          const bool whole = nh + 32 <= P.N;
          if (part) {
            for (int src = 0; src < W; ++src) {
              if (src == R) continue;
              const __nv_bfloat16* prow = part + (long long)src * Ms * P.N + nh;
              if (whole) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 raw = tp_ld_cg(prow + q * 8);
                  const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(hh[e]);
                    v[q * 8 + 2 * e] += f.x;
                    v[q * 8 + 2 * e + 1] += f.y;
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (nh + j < P.N) v[j] += __bfloat162float(prow[j]);
              }
            }
          }
          if (P.bias && (P.mode == 0 || part)) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nh + j < P.N) v[j] += __bfloat162float(P.bias[nh + j]);
          }
          if (part && P.residual) {
            const __nv_bfloat16* rrow = P.residual + ((long long)mbl * TP_BLOCK_M + row_in_tile) * P.ld_res + nh;
            if (whole) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 raw = *reinterpret_cast<const uint4*>(rrow + q * 8);
                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = __bfloat1622float2(hh[e]);
                  v[q * 8 + 2 * e] += f.x;
                  v[q * 8 + 2 * e + 1] += f.y;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nh + j < P.N) v[j] += __bfloat162float(rrow[j]);
            }
          }
          __nv_bfloat16* crow = (remote ? row_ptr + (long long)lane * P.N : row_ptr) + nh;
          if (whole) {
            uint4* d4 = reinterpret_cast<uint4*>(crow);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              d4[q] = w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nh + j < P.N) crow[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (remote) {
        // this warp's part of the tile is on its way to the owner: make it visible, then count it
        __threadfence_system();
        __syncwarp();
        if (lane == 0) tp_red_release_sys_add(P.flags_peer[dst] + 2 * W + mbl * W + R, 1);
      }
    }
  }

  // ---- common exit of the GEMM roles
  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }

}

template <int BLOCK_N, bool B_MN>
void tp_launch(const CUtensorMap& ta, const CUtensorMap& tag, const CUtensorMap& tb, const TpParams& p, int device,
               cudaStream_t stream) {
  using S = TpSmem<BLOCK_N>;
  auto kern = tp_gemm_kernel<BLOCK_N, B_MN>;
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  const int sms = sm_count(device);
  const int tiles = p.m_blocks * p.n_blocks;
  int grid = p.mode == 0 ? std::min(sms, tiles + p.n_comm) : std::min(sms, tiles);
  kern<<<grid, TP_THREADS, S::TOTAL, stream>>>(ta, tag, tb, p);
  RT_LAUNCH_CHECK();
}

}  // namespace

void tp_gemm(const TpGemmArgs& a, cudaStream_t stream) {
  RT_CHECK(a.mode == 0 || a.mode == 1, "tp_gemm: mode must be 0 (all-gather -> GEMM) or 1 (GEMM -> reduce-scatter)");
  RT_CHECK(a.world >= 1 && a.world <= RT_MAX_PEERS && a.rank >= 0 && a.rank < a.world, "tp_gemm: bad world / rank");
  RT_CHECK(a.rows_per_rank > 0 && a.rows_per_rank % TP_BLOCK_M == 0, "tp_gemm: rows per rank must be a multiple of 128");
  RT_CHECK(a.K % 8 == 0 && a.N % 8 == 0, "tp_gemm: K and N must be multiples of 8");
  RT_CHECK(a.epoch >= 1, "tp_gemm: epoch counts from 1");
  const int device = current_device();
  TpParams p{};
  p.mode = a.mode;
  p.M = a.rows_per_rank * a.world;
  p.N = a.N;
  p.K = a.K;
  const int block_n = a.N <= 128 ? 128 : 256;
  p.mbs = a.rows_per_rank / TP_BLOCK_M;
  p.m_blocks = p.mbs * a.world;
  p.n_blocks = (a.N + block_n - 1) / block_n;
  p.k_blocks = (a.K + TP_BLOCK_K - 1) / TP_BLOCK_K;
  p.world = a.world;
  p.rank = a.rank;
  p.epoch = a.epoch;
  p.timeout_ns = a.timeout_ns;
  p.C = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.ldc = a.ld_out;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ld_res = a.ld_res;
  p.status = status_word(device);
  for (int r = 0; r < a.world; ++r) {
    p.flags_peer[r] = a.flags[r];
    p.x_peer[r] = reinterpret_cast<const __nv_bfloat16*>(a.x_shards[r]);
    p.stage_peer[r] = reinterpret_cast<__nv_bfloat16*>(a.stage[r]);
  }
  CUtensorMap ta, tag;
  if (a.mode == 0) {
    RT_CHECK(a.x_shards[a.rank] && a.gather && a.mb_ready && a.comm_done, "tp_gemm(AG): missing buffers");
    const int sms = sm_count(device);
    p.n_comm = a.world > 1 ? std::max(1, std::min(a.n_comm > 0 ? a.n_comm : 8, sms / 4)) : 1;
    p.xg = reinterpret_cast<__nv_bfloat16*>(a.gather);
    p.mb_ready = a.mb_ready;
    p.comm_done = a.comm_done;
    ta = make_tmap_2byte(a.x_shards[a.rank], a.K, a.rows_per_rank, 1, a.K, 0, 64, TP_BLOCK_M);
    tag = make_tmap_2byte(a.gather, a.K, p.M, 1, a.K, 0, 64, TP_BLOCK_M);
  } else {
    RT_CHECK(a.x && a.stage[a.rank], "tp_gemm(RS): missing buffers");
    p.stage_parity_stride = (long long)a.world * a.rows_per_rank * a.N;
    ta = make_tmap_2byte(a.x, a.K, p.M, 1, a.ld_x, 0, 64, TP_BLOCK_M);
    tag = ta;
  }
  const CUtensorMap tb = a.b_mn ? make_tmap_2byte(a.b, a.N, a.K, 1, a.ldb, 0, 64, 64)
                                : make_tmap_2byte(a.b, a.K, a.N, 1, a.ldb, 0, 64, block_n);
  if (block_n == 256) {
    if (a.b_mn) tp_launch<256, true>(ta, tag, tb, p, device, stream);
    else tp_launch<256, false>(ta, tag, tb, p, device, stream);
  } else {
    if (a.b_mn) tp_launch<128, true>(ta, tag, tb, p, device, stream);
    else tp_launch<128, false>(ta, tag, tb, p, device, stream);
  }
}

}  // namespace rt
