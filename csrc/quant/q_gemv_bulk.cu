// Dequant-fused Q4_0 / Q8_0 matrix-vector product fed by the bulk-copy engine (decode path, M <= 4 rows).
//
// Same math and device layout as q_gemv.cu.  The difference is how the weights reach the SM: a producer
// warp streams tiles of 32 output rows x 32 quant blocks (1024 weights per row) into a shared-memory ring
// with two tiled TMA loads per stage (`cp.async.bulk.tensor.2d`: the nibbles as a 32-row box of 32-bit
// words, the scales as a 32 x 32 box of halves; per-row 1-D bulk copies were tried first and were bound by
// the copy engine's request rate) that complete on an mbarrier, and eight consumer warps (four rows each) expand and multiply out of shared memory.
// With 6 stages of 18 KB in flight per CTA and two CTAs per SM, about 200 KB per SM is always on its way
// from HBM regardless of what the consumer warps are doing, which is what a latency-bound register-fed
// GEMV (one or two 16-byte loads per lane in flight) cannot reach.  CTAs are persistent over row tiles.
//
// Waits are bounded (mbar_wait): on a timeout the CTA sets its abort flag and the per-device status
// word, the producer stops issuing and waits for the copies it has in flight, and every role falls
// through to the common exit.
//
// Requirements: K a multiple of 256 (so that a row of scales is a 16-byte multiple, which a tensor map
// needs) and 16-byte aligned x rows; other shapes take the register-fed kernel.  Boxes that reach past
// the last row or the last block read as zero and still count their full size on the mbarrier.
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "q_expand.cuh"

namespace rt {

namespace {

constexpr int QB_KB = 32;      // quant blocks per tile and row (one per consumer lane)
constexpr int QB_CONS = 8;     // consumer warps; each owns RPW rows of a tile of QB_CONS * RPW rows
constexpr int QB_THREADS = (QB_CONS + 1) * 32;

// RPW = rows per consumer warp (tiles of QB_CONS * RPW = 32 rows).
template <bool Q8, int RPW>
struct QbCfg {
  static constexpr int ROWS = QB_CONS * RPW;
  static constexpr int BQ = Q8 ? 32 : 16;                         // quant bytes per block
  static constexpr int Q_BYTES = ROWS * QB_KB * BQ;               // 16 KB / 32 KB at 32 rows
  static constexpr int S_BYTES = ROWS * QB_KB * 2;                // 2 KB at 32 rows
  static constexpr int STAGE_BYTES = Q_BYTES + S_BYTES;
  static constexpr int STAGES = (Q8 && RPW == 4) ? 4 : 6;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STAGES * 8 + 16;
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

template <bool Q8, int M, int RPW>
__global__ void __launch_bounds__(QB_THREADS) q_gemv_bulk_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                 const __grid_constant__ CUtensorMap tmap_s,
                                                                 const __half* __restrict__ x, long long ldx,
                                                                 __half* __restrict__ y, long long ldy,
                                                                 const __half* __restrict__ bias,
                                                                 const __half* __restrict__ residual, long long ldr,
                                                                 int N, int K, int* status) {
  using Cfg = QbCfg<Q8, RPW>;
  constexpr int QB_ROWS = Cfg::ROWS;
  constexpr int QB_RPW = RPW;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + Cfg::STAGES;
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(empty + Cfg::STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = K >> 5;
  const int k_tiles = (nb + QB_KB - 1) / QB_KB;
  const int row_tiles = (N + QB_ROWS - 1) / QB_ROWS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], QB_CONS);
    }
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_s);
  }
  __syncthreads();

  if (warp == QB_CONS) {
    // ------------------------------------------------------------------ producer (one elected lane issues)
    uint32_t it = 0;
    bool ok = true;
    for (int rt = blockIdx.x; rt < row_tiles && ok; rt += gridDim.x) {
      for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        if (it >= (uint32_t)Cfg::STAGES) ok = mbar_wait(&empty[s], ph ^ 1, ctl, status, RT_ERR_TIMEOUT_PRODUCER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int kb0 = kt * QB_KB;
        uint8_t* sq = smem + s * Cfg::STAGE_BYTES;
        uint8_t* ss = sq + Cfg::Q_BYTES;
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[s], (uint32_t)Cfg::STAGE_BYTES);
          tma_load_2d(sq, &tmap_q, &full[s], kb0 * (Cfg::BQ / 4), rt * QB_ROWS);
          tma_load_2d(ss, &tmap_s, &full[s], kb0, rt * QB_ROWS);
        }
        __syncwarp();
      }
    }
    // Copies still in flight must land before the CTA may exit: wait for the last armed phase of every stage.
    if (lane == 0) {
      const uint32_t armed = it < (uint32_t)Cfg::STAGES ? it : (uint32_t)Cfg::STAGES;
      for (uint32_t j = 0; j < armed; ++j) {
        const uint32_t i2 = it - 1 - j;
        mbar_wait(&full[i2 % Cfg::STAGES], (i2 / Cfg::STAGES) & 1, ctl, nullptr, 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    uint32_t it = 0;
    bool ok = true;
    for (int rt = blockIdx.x; rt < row_tiles && ok; rt += gridDim.x) {
      float acc[QB_RPW][M];
#pragma unroll
      for (int r = 0; r < QB_RPW; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
      for (int kt = 0; kt < k_tiles; ++kt, ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        ok = mbar_wait(&full[s], ph, ctl, status, RT_ERR_TIMEOUT_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int kb0 = kt * QB_KB;
        const int nblk = min(QB_KB, nb - kb0);
        const uint8_t* sq = smem + s * Cfg::STAGE_BYTES;
        const __half* ss = reinterpret_cast<const __half*>(sq + Cfg::Q_BYTES);
        if (lane < nblk) {
          __half2 xh[M][16];
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(x + m * ldx + ((long long)(kb0 + lane) << 5));
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(&xh[m][4 * i]) = __ldg(xp + i);
          }
#pragma unroll
          for (int r = 0; r < QB_RPW; ++r) {
            const int row = warp * QB_RPW + r;
            const uint4* src = reinterpret_cast<const uint4*>(sq + (row * QB_KB + lane) * Cfg::BQ);
            __half2 w[16];
            if (Q8) expand_q8(src[0], src[Q8 ? 1 : 0], w);
            else expand_q4(src[0], w);
            const float d = __half2float(ss[row * QB_KB + lane]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              __half2 s0 = __float2half2_rn(0.f), s1 = __float2half2_rn(0.f);
#pragma unroll
              for (int j = 0; j < 16; j += 2) {
                s0 = __hfma2(w[j], xh[m][j], s0);
                s1 = __hfma2(w[j + 1], xh[m][j + 1], s1);
              }
              const float2 f = __half22float2(__hadd2(s0, s1));
              acc[r][m] = fmaf(d, f.x + f.y, acc[r][m]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      if (!ok) break;
#pragma unroll
      for (int r = 0; r < QB_RPW; ++r) {
        const int n = rt * QB_ROWS + warp * QB_RPW + r;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float v = warp_sum_f(acc[r][m]);
          if (lane == 0 && n < N) {
            if (bias) v += __half2float(bias[n]);
            if (residual) v += __half2float(residual[m * ldr + n]);
            y[m * ldy + n] = __float2half(v);
          }
        }
      }
    }
  }
  __syncthreads();
}

template <bool Q8, int M, int RPW>
void launch_bulk(const QGemvArgs& a, int m0, cudaStream_t s) {
  using Cfg = QbCfg<Q8, RPW>;
  constexpr int QB_ROWS = Cfg::ROWS;
  static bool attr_set[64] = {};  // per device
  auto kern = q_gemv_bulk_kernel<Q8, M, RPW>;
  const int dev = current_device();
  if (!attr_set[dev & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    attr_set[dev & 63] = true;
  }
  const int row_tiles = (a.N + QB_ROWS - 1) / QB_ROWS;
  const int ctas_per_sm = std::max(1, std::min(4, (224 * 1024) / Cfg::SMEM));
  const int grid = std::min(row_tiles, sm_count(dev) * ctas_per_sm);
  const __half* x = reinterpret_cast<const __half*>(a.x) + (long long)m0 * a.ldx;
  __half* y = reinterpret_cast<__half*>(a.y) + (long long)m0 * a.ldy;
  const __half* r = a.residual ? reinterpret_cast<const __half*>(a.residual) + (long long)m0 * a.ldr : nullptr;
  const uint64_t nb = a.K / 32;
  const CUtensorMap tq = make_tmap_rows(a.qs, 4, nb * (Cfg::BQ / 4), a.N, QB_KB * (Cfg::BQ / 4), QB_ROWS);
  const CUtensorMap ts = make_tmap_rows(a.scales, 2, nb, a.N, QB_KB, QB_ROWS);
  kern<<<grid, QB_THREADS, Cfg::SMEM, s>>>(tq, ts, x, a.ldx, y, a.ldy, reinterpret_cast<const __half*>(a.bias), r, a.ldr, a.N,
                                           a.K, status_word(dev));
  RT_LAUNCH_CHECK();
}

template <bool Q8, int RPW>
void dispatch_m(const QGemvArgs& a, int m0, int m, cudaStream_t s) {
  switch (m) {
    case 1: launch_bulk<Q8, 1, RPW>(a, m0, s); break;
    case 2: launch_bulk<Q8, 2, RPW>(a, m0, s); break;
    case 3: launch_bulk<Q8, 3, RPW>(a, m0, s); break;
    default: launch_bulk<Q8, 4, RPW>(a, m0, s); break;
  }
}

template <bool Q8>
void dispatch_rows(const QGemvArgs& a, int m0, int m, cudaStream_t s) {
  dispatch_m<Q8, 4>(a, m0, m, s);
}

}  // namespace

// Measured on B200 at the llama-7B shapes (benchmarks/kernel_bench.py --op qgemv): both kernels are bound by
// the dequantisation arithmetic, not by memory, at about 2.9 TB/s for one activation row; the ring wins
// (+10 to +20 %) for 3-4 rows when N gives at least two tiles per SM, the register kernel otherwise.
bool q_gemv_bulk_preferred(const QGemvArgs& a) {
  return a.M >= 3 && a.N >= 2 * 32 * sm_count(current_device());
}

bool q_gemv_bulk_supported(const QGemvArgs& a) {
  return a.K % 256 == 0 && a.ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.qs) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 15) == 0 && a.N >= 1;
}

// Rows of x are processed four at a time (each pass streams the weights once).
void q_gemv_bulk(const QGemvArgs& a, cudaStream_t stream) {
  RT_CHECK(q_gemv_bulk_supported(a), "q_gemv_bulk: unsupported shape or alignment");
  if (a.M == 0) return;
  for (int m0 = 0; m0 < a.M; m0 += 4) {
    const int m = std::min(4, a.M - m0);
    if (a.q8) dispatch_rows<true>(a, m0, m, stream);
    else dispatch_rows<false>(a, m0, m, stream);
  }
}

}  // namespace rt
