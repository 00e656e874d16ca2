// int8 x int8 -> int32 GEMM on the tcgen05 integer tensor cores (kind::i8), with an optional fused dequantisation
// epilogue:
//     acc[m][n]  = sum_k A[m][k] * B[n][k]                    A: s8 [M][K], B: s8 [N][K] (both K-major), acc s32 in TMEM
//     C_i32      = acc                                         (raw accumulator), or
//     C_f32      = acc * row_scale[m] * col_scale[n] + bias[n] (per-tensor scales: one-element arrays with stride 0)
// One CTA computes one 128 x 128 tile: warp 0 streams 128-byte K slices of A and B through a 4-stage TMA ring, warp 1
// issues tcgen05.mma (32 k per instruction), warps 2-5 read the accumulator with tcgen05.ld and store it.  int4
// operands are the same kernel on codes widened to one byte each.
// The reference names qmatmul_cuda / qconv2d_cuda but runs CPU loops behind them
// (src/quantization/hardware/cuda.rs:12-70, src/quantization/operations.rs:12-480).
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

constexpr int I8_BM = 128, I8_BN = 128, I8_BK = 128;  // BK in bytes = int8 elements: one 128-byte swizzle row
constexpr int I8_STAGES = 4;
constexpr int I8_THREADS = 192;

struct GemmI8Params {
  int M, N, K, k_blocks;
  int32_t* c_i32;
  float* c_f32;
  long long ldc;
  const float* row_scale;
  const float* col_scale;
  const float* bias;
  int row_scale_stride, col_scale_stride;  // 0: one scale for the whole tensor
  int* status;
};

struct GemmI8Smem {
  static constexpr int A_BYTES = I8_BM * I8_BK;
  static constexpr int B_BYTES = I8_BN * I8_BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = I8_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * I8_STAGES + 1) * 8 + 16;
};

// Instruction descriptor for kind::i8: D = s32 (2 at [4,6)), A / B = s8 (1 at [7,10) / [10,13)), both K-major.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_i8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(I8_THREADS, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmI8Params p) {
  using S = GemmI8Smem;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + I8_STAGES;
  uint64_t* acc_full = empty_bar + I8_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = I8_BN;
  const int mb = blockIdx.y, nb = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < I8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        const int s = kb % I8_STAGES;
        const uint32_t ph = (kb / I8_STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) break;
        uint8_t* sa = smem + s * S::STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
        // the maps describe the int8 rows as rows of 16-bit words: x counts words (64 words = 128 bytes)
        tma_load_3d(sa, &tmap_a, &full_bar[s], kb * (I8_BK / 2), mb * I8_BM, 0);
        tma_load_3d(sa + S::A_BYTES, &tmap_b, &full_bar[s], kb * (I8_BK / 2), nb * I8_BN, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(I8_BM, I8_BN);
      bool ok = true;
      for (int kb = 0; kb < p.k_blocks && ok; ++kb) {
        const int s = kb % I8_STAGES;
        const uint32_t ph = (kb / I8_STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < I8_BK / 32; ++kk)  // 32 int8 = 32 bytes per instruction
          umma_i8_ss(tmem_base, make_smem_desc_sw128(sa + kk * 32, 16, 1024), make_smem_desc_sw128(sb + kk * 32, 16, 1024), idesc,
                     (kb > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int m = mb * I8_BM + quarter * 32 + lane;
    if (mbar_wait(acc_full, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      const float rs = (p.c_f32 && m < p.M) ? p.row_scale[(long long)m * p.row_scale_stride] : 1.f;
#pragma unroll 1
      for (int c = 0; c < I8_BN / 32; ++c) {
        const int n0 = nb * I8_BN + c * 32;
        if (n0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + c * 32 + (uint32_t(quarter * 32) << 16), r);
        tmem_ld_wait();
        if (m >= p.M) continue;
        if (p.c_f32) {
          float* crow = p.c_f32 + (long long)m * p.ldc + n0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (n0 + j < p.N) {
              float v = float(int32_t(r[j])) * rs * p.col_scale[(long long)(n0 + j) * p.col_scale_stride];
              if (p.bias) v += p.bias[n0 + j];
              crow[j] = v;
            }
          }
        } else {
          int32_t* crow = p.c_i32 + (long long)m * p.ldc + n0;
          if (n0 + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              reinterpret_cast<uint4*>(crow)[q] = make_uint4(r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) crow[j] = int32_t(r[j]);
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

void gemm_i8(const GemmI8Args& g, cudaStream_t stream) {
  if (g.M == 0 || g.N == 0) return;
  RT_CHECK(g.K > 0 && g.K % 16 == 0, "gemm_i8: K must be a positive multiple of 16 (TMA rows are 16-byte aligned)");
  RT_CHECK(g.lda % 16 == 0 && g.ldb % 16 == 0, "gemm_i8: row strides must be multiples of 16 bytes");
  RT_CHECK((g.c_i32 != nullptr) != (g.c_f32 != nullptr), "gemm_i8: exactly one of the int32 / fp32 outputs");
  RT_CHECK(g.c_f32 == nullptr || (g.row_scale && g.col_scale), "gemm_i8: the fp32 output needs both scale arrays");
  const int device = current_device();
  static bool configured[64] = {false};
  if (!configured[device]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(gemm_i8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmI8Smem::TOTAL));
    configured[device] = true;
  }
  GemmI8Params p{};
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.k_blocks = (g.K + I8_BK - 1) / I8_BK;
  p.c_i32 = g.c_i32;
  p.c_f32 = g.c_f32;
  p.ldc = g.ldc;
  p.row_scale = g.row_scale;
  p.col_scale = g.col_scale;
  p.bias = g.bias;
  p.row_scale_stride = g.row_scale_per_row ? 1 : 0;
  p.col_scale_stride = g.col_scale_per_col ? 1 : 0;
  p.status = status_word(device);
  // int8 rows seen as rows of 16-bit words; parts of a box beyond K or beyond the last row read as zero
  CUtensorMap ta = make_tmap_2byte(g.a, uint64_t(g.K / 2), uint64_t(g.M), 1, uint64_t(g.lda / 2), 0, 64, I8_BM);
  CUtensorMap tb = make_tmap_2byte(g.b, uint64_t(g.K / 2), uint64_t(g.N), 1, uint64_t(g.ldb / 2), 0, 64, I8_BN);
  dim3 grid((g.N + I8_BN - 1) / I8_BN, (g.M + I8_BM - 1) / I8_BM);
  gemm_i8_tcgen05_kernel<<<grid, I8_THREADS, GemmI8Smem::TOTAL, stream>>>(ta, tb, p);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
