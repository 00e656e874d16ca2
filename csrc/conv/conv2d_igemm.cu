// Conv2d as implicit GEMM on tcgen05 (sm_100a), channels-last bf16.
//
//   forward  out[n,oh,ow,co] = sum_{kh,kw,ci} x[n, oh*s + kh - p, ow*s + kw - p, ci] * w[co,kh,kw,ci]  (+ bias)
//            GEMM view: M = output pixels, N = Cout, K = KH*KW*Cin.  No im2col buffer exists: the A tile of a
//            k-block (one filter tap, 64 input channels) is ONE rank-4 TMA box over the NHWC input, 64 channels x
//            TW x TH x TN output positions (TW*TH*TN = 128) read every `s` pixels starting at the tap's offset;
//            out-of-image positions (the padding halo) are zero-filled by the TMA unit.  The box lands in shared
//            memory as the same 128-row x 64-column swizzled K-major tile the plain GEMM uses, so the MMA loop,
//            TMEM double buffering and epilogue structure are those of gemm_tcgen05.cu.
//   dgrad    (stride 1) is the same kernel on dy with the filter rotated by 180 degrees and in/out channels swapped
//            (the Python side prepares that small tensor), padding KH-1-p.
//   wgrad    dw[co,kh,kw,ci] = sum_{n,oh,ow} dy[n,oh,ow,co] * x[n, oh*s + kh - p, ow*s + kw - p, ci]
//            GEMM view: M = Cout, N = Cin, K = output pixels, per tap.  Both operands are read "MN-major" (pixels are
//            the reduction dim): A boxes come from dy, B boxes from x with the tap offset; the pixel range is split
//            over CTAs and partial tiles are added to the fp32 gradient with float4 atomics.
//
// The reference's convolution is nested host loops (src/nn/conv2d.rs:150-260) and an im2col CUDA-C string kernel
// followed by SGEMM (K9-K12, src/gpu/conv_ops.rs:27-765).  Requirements here: Cin % 64 == 0 (forward / wgrad B
// boxes are 64 channels wide), Cout % 8 == 0; other layers (the 3-channel stem) stay on the library path.
#include <cstdlib>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

constexpr int CV_THREADS = 320;
constexpr int CV_BK = 64;

struct ConvParams {
  int N, H, W, Cin, OH, OW, Cout, KH, KW, stride, pad, pad_h;  // pad: along W; pad_h: along H
  int TW, TH, TN, tiles_w, tiles_h, tiles_n;  // output-pixel tile and tile counts
  int m_tiles, n_blocks, k_chunks;            // k_chunks = Cin / 64
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  long long out_sn, out_sh, out_sw;  // element strides of the output view
  // wgrad
  float* dw;       // [Cout][KH*KW][Cin] fp32, accumulated into
  int split;       // CTAs per output tile along the pixel dimension
  int* status;
};

template <int BLOCK_N>
struct ConvSmem {
  static constexpr int A_BYTES = 128 * CV_BK * 2;
  static constexpr int B_BYTES = BLOCK_N * CV_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ void cv_decode(int t, const ConvParams& p, int& mt, int& nb) {
  constexpr int GROUP = 8;
  const int band = GROUP * p.n_blocks;
  const int g = t / band, first = g * GROUP;
  const int rows = min(GROUP, p.m_tiles - first);
  const int in_band = t - g * band;
  mt = first + in_band % rows;
  nb = in_band / rows;
}

__device__ __forceinline__ void cv_tile_origin(int mt, const ConvParams& p, int& n0, int& oh0, int& ow0) {
  const int tw = mt % p.tiles_w;
  const int th = (mt / p.tiles_w) % p.tiles_h;
  const int tn = mt / (p.tiles_w * p.tiles_h);
  n0 = tn * p.TN;
  oh0 = th * p.TH;
  ow0 = tw * p.TW;
}

// ------------------------------------------------------------------------------------------ forward / dgrad
template <int BLOCK_N>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_fwd_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const ConvParams p) {
  using S = ConvSmem<BLOCK_N>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;

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
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = p.m_tiles * p.n_blocks;
  const int k_blocks = p.KH * p.KW * p.k_chunks;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mt, nb, n0, oh0, ow0;
        cv_decode(t, p, mt, nb);
        cv_tile_origin(mt, p, n0, oh0, ow0);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const int tap = kb / p.k_chunks, cc = kb - tap * p.k_chunks;
          const int kh = tap / p.KW, kw = tap - kh * p.KW;
          uint8_t* sa = smem + s * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_4d(sa, &tmap_x, &full_bar[s], cc * CV_BK, ow0 * p.stride + kw - p.pad, oh0 * p.stride + kh - p.pad_h, n0);
          tma_load_3d(sb, &tmap_w, &full_bar[s], tap * p.Cin + cc * CV_BK, nb * BLOCK_N, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, BLOCK_N, false, false, true);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < CV_BK / 16; ++kk)
            umma_f16_ss(d_tmem, make_smem_desc_sw128(sa + kk * 32, 16, 1024), make_smem_desc_sw128(sb + kk * 32, 16, 1024), idesc,
                        (kb > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;  // row of the tile = position in the TMA box: ((tn * TH) + th) * TW + tw
    const int tw = r % p.TW, th = (r / p.TW) % p.TH, tn = r / (p.TW * p.TH);
    uint32_t tile_i = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
      int mt, nb, n0, oh0, ow0;
      cv_decode(t, p, mt, nb);
      cv_tile_origin(mt, p, n0, oh0, ow0);
      const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int n = n0 + tn, oh = oh0 + th, ow = ow0 + tw;
      const bool row_ok = n < p.N && oh < p.OH && ow < p.OW;
      __nv_bfloat16* orow = p.out + n * p.out_sn + oh * p.out_sh + ow * p.out_sw;
#pragma unroll 1
      for (int c = col_half * (BLOCK_N / 64); c < (col_half + 1) * (BLOCK_N / 64); ++c) {
        const int c0 = nb * BLOCK_N + c * 32;
        if (c0 >= p.Cout) break;
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + acc * BLOCK_N + c * 32 + (uint32_t(quarter * 32) << 16), v);
        tmem_ld_wait();
        if (row_ok) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.Cout) f[j] += __bfloat162float(p.bias[c0 + j]);
          }
          if (c0 + 32 <= p.Cout) {
            uint4* d4 = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(f[q * 8 + 0], f[q * 8 + 1]);
              w.y = pack_bf16x2(f[q * 8 + 2], f[q * 8 + 3]);
              w.z = pack_bf16x2(f[q * 8 + 4], f[q * 8 + 5]);
              w.w = pack_bf16x2(f[q * 8 + 6], f[q * 8 + 7]);
              d4[q] = w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.Cout) orow[c0 + j] = __float2bfloat16(f[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
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

// ------------------------------------------------------------------------------- forward, resident halo
// 3 x 3, stride 1, padding 1, 64 input channels: the general kernel above fetches the input tile once per filter
// tap (nine boxes per output tile), which makes the 64-channel layers L2 -> shared-memory bound.  Here the image
// is read as rows that are two pixels wider than the image (the TMA box starts at column -1 and zero-fills the
// border), so in the flattened, padded pixel order q = row * (W + 2) + col the tap (kh, kw) of output q is
// input q + kh (W + 2) + kw: every tap's A operand is the SAME shared-memory halo tile, shifted by whole
// 128-byte pixel rows.  One box per tile (all rows the 128 outputs touch), nine descriptor offsets, and the
// 9 x BLOCK_N x 64 filter stays resident in shared memory for the CTA's lifetime.  Outputs that fall on the
// two padding columns are computed and dropped (2 / (W + 2) of the tile).
struct HaloParams {
  int N, H, W, Cout, PW, R;          // PW = W + 2, R = rows per halo box
  int tiles_per_img, n_blocks;
  int halo_bytes, stages;            // bytes of one halo stage (multiple of 1024)
  int base_offset_mode;              // 1: descriptors carry (address >> 7) & 7 as the matrix base offset
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  long long out_sn, out_sh, out_sw;
  int* status;
};

__device__ __forceinline__ uint64_t make_smem_desc_sw128_rows(uint32_t smem_addr, int base_offset_mode) {
  uint64_t d = make_smem_desc_sw128(smem_addr, 16, 1024);
  if (base_offset_mode) d |= static_cast<uint64_t>((smem_addr >> 7) & 7) << 49;
  return d;
}

template <int BLOCK_N>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_fwd_halo_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const HaloParams p) {
  constexpr int W_BYTES = 9 * BLOCK_N * 128;
  constexpr int MAX_STAGES = 4;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint8_t* halo = smem + W_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(halo + (size_t)p.stages * p.halo_bytes);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* tmem_full = empty_bar + MAX_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* w_bar = tmem_empty + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(w_bar + 1);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;
  const int STAGES = p.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    mbar_init(w_bar, 1);
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // a CTA keeps one block of output channels (its filter stays resident) and walks the pixel tiles
  const int nb = (int)blockIdx.x % p.n_blocks;
  const int first = (int)blockIdx.x / p.n_blocks, step = (int)gridDim.x / p.n_blocks;
  const int m_tiles = p.N * p.tiles_per_img;

  if (warp == 0) {
    if (lane == 0 && first < m_tiles) {
      mbar_arrive_expect_tx(w_bar, W_BYTES);
      for (int tap = 0; tap < 9; ++tap) tma_load_3d(smem + tap * BLOCK_N * 128, &tmap_w, w_bar, tap * 64, nb * BLOCK_N, 0);
      uint32_t it = 0;
      for (int mt = first; mt < m_tiles; mt += step, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) break;
        const int n = mt / p.tiles_per_img, p0 = (mt - n * p.tiles_per_img) * 128;
        mbar_arrive_expect_tx(&full_bar[s], (uint32_t)p.R * p.PW * 128);
        tma_load_4d(halo + (size_t)s * p.halo_bytes, &tmap_x, &full_bar[s], 0, -1, p0 / p.PW - 1, n);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && first < m_tiles) {
      constexpr uint32_t idesc = make_idesc_f16(128, BLOCK_N, false, false, true);
      bool ok = mbar_wait(w_bar, 0, ctl, p.status, RT_ERR_TIMEOUT_MMA);
      uint32_t it = 0;
      for (int mt = first; mt < m_tiles && ok; mt += step, ++it) {
        const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_MMA) ||
            !mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int p0 = (mt % p.tiles_per_img) * 128;
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        const uint32_t sh = smem_u32(halo + (size_t)s * p.halo_bytes) + (uint32_t)(p0 % p.PW) * 128;
        const uint32_t sw = smem_u32(smem);
#pragma unroll 1
        for (int tap = 0; tap < 9; ++tap) {
          const int kh = tap / 3, kw = tap - kh * 3;
          const uint32_t sa = sh + (uint32_t)(kh * p.PW + kw) * 128;
          const uint32_t sb = sw + tap * BLOCK_N * 128;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ss(d_tmem, make_smem_desc_sw128_rows(sa + kk * 32, p.base_offset_mode), make_smem_desc_sw128(sb + kk * 32, 16, 1024),
                        idesc, (tap > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
        umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    uint32_t it = 0;
    for (int mt = first; mt < m_tiles; mt += step, ++it) {
      const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int n = mt / p.tiles_per_img, q = (mt - n * p.tiles_per_img) * 128 + r;
      const int oh = q / p.PW, ow = q - oh * p.PW;
      const bool row_ok = oh < p.H && ow < p.W;
      __nv_bfloat16* orow = p.out + n * p.out_sn + oh * p.out_sh + ow * p.out_sw;
#pragma unroll 1
      for (int c = col_half * (BLOCK_N / 64); c < (col_half + 1) * (BLOCK_N / 64); ++c) {
        const int c0 = nb * BLOCK_N + c * 32;
        if (c0 >= p.Cout) break;
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + acc * BLOCK_N + c * 32 + (uint32_t(quarter * 32) << 16), v);
        tmem_ld_wait();
        if (row_ok) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] += __bfloat162float(p.bias[c0 + j]);
          }
          uint4* d4 = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            uint4 w;
            w.x = pack_bf16x2(f[qd * 8 + 0], f[qd * 8 + 1]);
            w.y = pack_bf16x2(f[qd * 8 + 2], f[qd * 8 + 3]);
            w.z = pack_bf16x2(f[qd * 8 + 4], f[qd * 8 + 5]);
            w.w = pack_bf16x2(f[qd * 8 + 6], f[qd * 8 + 7]);
            d4[qd] = w;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
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

// ------------------------------------------------------------------------------------------ wgrad
// One CTA = one output tile (128 out-channels x BLOCK_N in-channels of one tap) x one slice of the pixel tiles.
// k-block = 64 output pixels (TW*TH*TN = 64).
template <int BLOCK_N>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x, const ConvParams p) {
  using S = ConvSmem<BLOCK_N>;  // A: [64 pixels][128 co] as two 64-column chunks (16 KB) ; B: [64 pixels][BLOCK_N ci]
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_full + 4);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = BLOCK_N < 32 ? 32 : BLOCK_N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // blockIdx.x = output tile (co block, tap, ci block), blockIdx.y = pixel slice
  const int ci_blocks = (p.Cin + BLOCK_N - 1) / BLOCK_N;
  const int taps = p.KH * p.KW;
  const int cib = blockIdx.x % ci_blocks;
  const int tap = (blockIdx.x / ci_blocks) % taps;
  const int cob = blockIdx.x / (ci_blocks * taps);
  const int kh = tap / p.KW, kw = tap - kh * p.KW;
  const int per = (p.m_tiles + p.split - 1) / p.split;
  const int mt0 = blockIdx.y * per, mt1 = min(p.m_tiles, mt0 + per);
  const int n_kb = max(0, mt1 - mt0);

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        int n0, oh0, ow0;
        cv_tile_origin(mt0 + i, p, n0, oh0, ow0);
        uint8_t* sa = smem + s * S::STAGE_BYTES;
        uint8_t* sb = sa + S::A_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], S::A_BYTES + BLOCK_N * 64 * 2);
#pragma unroll
        for (int c = 0; c < 2; ++c) tma_load_4d(sa + c * 8192, &tmap_dy, &full_bar[s], cob * 128 + c * 64, ow0, oh0, n0);
#pragma unroll
        for (int c = 0; c < BLOCK_N / 64; ++c)
          tma_load_4d(sb + c * 8192, &tmap_x, &full_bar[s], cib * BLOCK_N + c * 64, ow0 * p.stride + kw - p.pad,
                      oh0 * p.stride + kh - p.pad_h, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kb > 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, BLOCK_N, true, true, true);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < CV_BK / 16; ++kk)
          umma_f16_ss(tmem_base, make_smem_desc_sw128(sa + kk * 2048, 8192, 1024), make_smem_desc_sw128(sb + kk * 2048, 8192, 1024),
                      idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(tmem_full);
    }
  } else if (n_kb > 0) {
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const int co = cob * 128 + quarter * 32 + lane;
    if (mbar_wait(tmem_full, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      constexpr int CHUNKS = BLOCK_N / 32;  // 2 or 4
#pragma unroll 1
      for (int c = col_half * (CHUNKS / 2); c < (col_half + 1) * (CHUNKS / 2); ++c) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + c * 32 + (uint32_t(quarter * 32) << 16), v);
        tmem_ld_wait();
        const int ci0 = cib * BLOCK_N + c * 32;
        if (co < p.Cout && ci0 < p.Cin) {
          float4* dst = reinterpret_cast<float4*>(p.dw + ((long long)co * taps + tap) * p.Cin + ci0);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            atomicAdd(dst + q, make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]),
                                           __uint_as_float(v[q * 4 + 3])));
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

// Three-tap variant for KW == 3: one CTA owns 128 out-channels x 64 in-channels x the three taps of one kernel ROW.
// The three input boxes (shifted by one pixel in W) sit side by side as three 64-column chunks of one MN-major B tile,
// so one MMA of N = 192 serves them and the dy tile is fetched once per three taps instead of once per tap
// (the kernel is bound by L2 -> shared-memory traffic, not by the tensor pipe).
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_wgrad3_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x, const ConvParams p) {
  constexpr int BLOCK_N = 192;   // 3 taps x 64 in-channels
  using S = ConvSmem<256>;       // A: [64 pixels][128 co] (16 KB); B: three [64 pixels][64 ci] chunks (24 of 32 KB)
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_full + 4);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_base_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    ctl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // blockIdx.x = output tile (co block, kernel row, 64-channel ci block), blockIdx.y = pixel slice
  const int ci_blocks = p.Cin / 64;
  const int taps = p.KH * p.KW;
  const int cib = blockIdx.x % ci_blocks;
  const int kh = (blockIdx.x / ci_blocks) % p.KH;
  const int cob = blockIdx.x / (ci_blocks * p.KH);
  const int per = (p.m_tiles + p.split - 1) / p.split;
  const int mt0 = blockIdx.y * per, mt1 = min(p.m_tiles, mt0 + per);
  const int n_kb = max(0, mt1 - mt0);

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        int n0, oh0, ow0;
        cv_tile_origin(mt0 + i, p, n0, oh0, ow0);
        uint8_t* sa = smem + s * S::STAGE_BYTES;
        uint8_t* sb = sa + S::A_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], S::A_BYTES + BLOCK_N * 64 * 2);
#pragma unroll
        for (int c = 0; c < 2; ++c) tma_load_4d(sa + c * 8192, &tmap_dy, &full_bar[s], cob * 128 + c * 64, ow0, oh0, n0);
#pragma unroll
        for (int kw = 0; kw < 3; ++kw)      // chunk kw of the B tile = the box of tap (kh, kw)
          tma_load_4d(sb + kw * 8192, &tmap_x, &full_bar[s], cib * 64, ow0 * p.stride + kw - p.pad, oh0 * p.stride + kh - p.pad_h, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kb > 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, BLOCK_N, true, true, true);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < CV_BK / 16; ++kk)
          umma_f16_ss(tmem_base, make_smem_desc_sw128(sa + kk * 2048, 8192, 1024), make_smem_desc_sw128(sb + kk * 2048, 8192, 1024),
                      idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(tmem_full);
    }
  } else if (n_kb > 0) {
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const int co = cob * 128 + quarter * 32 + lane;
    if (mbar_wait(tmem_full, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      constexpr int CHUNKS = BLOCK_N / 32;  // 6: two 32-column chunks per tap
#pragma unroll 1
      for (int c = col_half * (CHUNKS / 2); c < (col_half + 1) * (CHUNKS / 2); ++c) {
        const int tap = kh * p.KW + (c >> 1);
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_base + c * 32 + (uint32_t(quarter * 32) << 16), v);
        tmem_ld_wait();
        const int ci0 = cib * 64 + (c & 1) * 32;
        if (co < p.Cout && ci0 < p.Cin) {
          float4* dst = reinterpret_cast<float4*>(p.dw + ((long long)co * taps + tap) * p.Cin + ci0);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            atomicAdd(dst + q, make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]),
                                           __uint_as_float(v[q * 4 + 3])));
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

void pick_tile(int OH, int OW, int Nimg, int pixels, int& TW, int& TH, int& TN) {
  // widths of 8 or 16 output columns, whichever wastes fewer columns; then rows, then images
  const int w8 = (OW + 7) / 8 * 8, w16 = (OW + 15) / 16 * 16;
  TW = (w8 <= w16 && pixels / 8 >= 1) ? 8 : 16;
  if (TW > pixels) TW = pixels;
  int th = 1;
  while (th * 2 <= pixels / TW && th < OH) th *= 2;
  TH = th;
  TN = pixels / (TW * TH);
  (void)Nimg;
}

void fill_common(const Conv2dArgs& a, ConvParams& p, int pixels) {
  p.N = a.N; p.H = a.H; p.W = a.W; p.Cin = a.Cin; p.Cout = a.Cout; p.KH = a.KH; p.KW = a.KW; p.stride = a.stride; p.pad = a.pad;
  p.pad_h = a.pad_h >= 0 ? a.pad_h : a.pad;
  p.OH = a.out_h > 0 ? a.out_h : (a.H + 2 * p.pad_h - a.KH) / a.stride + 1;
  p.OW = a.out_w > 0 ? a.out_w : (a.W + 2 * a.pad - a.KW) / a.stride + 1;
  p.out_sw = a.out_sw > 0 ? a.out_sw : a.Cout;
  p.out_sh = a.out_sh > 0 ? a.out_sh : (long long)p.OW * a.Cout;
  p.out_sn = a.out_sn > 0 ? a.out_sn : (long long)p.OH * p.OW * a.Cout;
  pick_tile(p.OH, p.OW, a.N, pixels, p.TW, p.TH, p.TN);
  p.tiles_w = (p.OW + p.TW - 1) / p.TW;
  p.tiles_h = (p.OH + p.TH - 1) / p.TH;
  p.tiles_n = (a.N + p.TN - 1) / p.TN;
  p.m_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
  p.k_chunks = a.Cin / 64;
}

void check_conv(const Conv2dArgs& a) {
  RT_CHECK(a.Cin % 64 == 0, "conv2d_igemm: input channels must be a multiple of 64");
  RT_CHECK(a.Cout % 8 == 0, "conv2d_igemm: output channels must be a multiple of 8");
  RT_CHECK(a.stride >= 1 && a.stride <= 4 && a.pad >= 0 && a.KH >= 1 && a.KW >= 1 && a.KH <= 7 && a.KW <= 7, "conv2d_igemm: unsupported geometry");
  RT_CHECK(a.N > 0 && (a.out_h > 0 || (a.H + 2 * (a.pad_h >= 0 ? a.pad_h : a.pad) >= a.KH && a.W + 2 * a.pad >= a.KW)), "conv2d_igemm: empty output");
  RT_CHECK(a.out_sw % 8 == 0 && a.out_sh % 8 == 0 && a.out_sn % 8 == 0, "conv2d_igemm: output strides must keep 16-byte alignment");
}

template <int BLOCK_N>
void launch_fwd(const Conv2dArgs& a, ConvParams& p, int device, cudaStream_t stream) {
  using S = ConvSmem<BLOCK_N>;
  auto kern = conv_fwd_kernel<BLOCK_N>;
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  p.n_blocks = (a.Cout + BLOCK_N - 1) / BLOCK_N;
  const CUtensorMap tx = make_tmap_nhwc(a.x, a.Cin, a.W, a.H, a.N, p.TW, p.TH, p.TN, a.stride);
  const CUtensorMap tw = make_tmap_2byte(a.w, (uint64_t)a.KH * a.KW * a.Cin, a.Cout, 1, (uint64_t)a.KH * a.KW * a.Cin, 0, 64, BLOCK_N);
  const int grid = std::min(p.m_tiles * p.n_blocks, sm_count(device));
  kern<<<grid, CV_THREADS, S::TOTAL, stream>>>(tx, tw, p);
  RT_LAUNCH_CHECK();
}

template <int BLOCK_N>
void launch_wgrad(const Conv2dArgs& a, ConvParams& p, int device, cudaStream_t stream) {
  using S = ConvSmem<BLOCK_N>;
  auto kern = conv_wgrad_kernel<BLOCK_N>;
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  const int out_tiles = ((a.Cout + 127) / 128) * a.KH * a.KW * ((a.Cin + BLOCK_N - 1) / BLOCK_N);
  const int sms = sm_count(device);
  p.split = std::max(1, std::min(p.m_tiles, (2 * sms + out_tiles - 1) / out_tiles));
  const CUtensorMap tdy = make_tmap_nhwc(a.dy, a.Cout, p.OW, p.OH, a.N, p.TW, p.TH, p.TN, 1);
  const CUtensorMap tx = make_tmap_nhwc(a.x, a.Cin, a.W, a.H, a.N, p.TW, p.TH, p.TN, a.stride);
  kern<<<dim3(out_tiles, p.split), CV_THREADS, S::TOTAL, stream>>>(tdy, tx, p);
  RT_LAUNCH_CHECK();
}

void launch_wgrad3(const Conv2dArgs& a, ConvParams& p, int device, cudaStream_t stream) {
  using S = ConvSmem<256>;
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(conv_wgrad3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  const int out_tiles = ((a.Cout + 127) / 128) * a.KH * (a.Cin / 64);
  const int sms = sm_count(device);
  p.split = std::max(1, std::min(p.m_tiles, (2 * sms + out_tiles - 1) / out_tiles));
  const CUtensorMap tdy = make_tmap_nhwc(a.dy, a.Cout, p.OW, p.OH, a.N, p.TW, p.TH, p.TN, 1);
  const CUtensorMap tx = make_tmap_nhwc(a.x, a.Cin, a.W, a.H, a.N, p.TW, p.TH, p.TN, a.stride);
  conv_wgrad3_kernel<<<dim3(out_tiles, p.split), CV_THREADS, S::TOTAL, stream>>>(tdy, tx, p);
  RT_LAUNCH_CHECK();
}

// 3 x 3 / stride 1 / pad 1 / 64 input channels / Cout a multiple of 64: the resident-halo kernel.  Returns false when
// the layer does not qualify or the tiles do not fit in shared memory (the general kernel takes it then).
// RUSTORCH_CONV_HALO: 0 = off, 1 (default) = on.  The shifted descriptors carry no matrix base offset: the tensor core
// applies the 128-byte swizzle to absolute shared-memory address bits, exactly as TMA wrote the tile (setting the
// base-offset field to (address >> 7) & 7 as well gives wrong results; mode 2 keeps that variant for reference).
template <int BLOCK_N>
bool launch_fwd_halo(const Conv2dArgs& a, const ConvParams& cp, int mode, int device, cudaStream_t stream) {
  HaloParams p{};
  p.N = a.N; p.H = a.H; p.W = a.W; p.Cout = a.Cout;
  p.PW = a.W + 2;
  p.R = (127 + 2 * p.PW + 2) / p.PW + 2;
  if (p.PW > 256 || p.R > 256) return false;
  p.tiles_per_img = (a.H * p.PW + 127) / 128;
  p.n_blocks = a.Cout / BLOCK_N;
  p.halo_bytes = ((p.R * p.PW * 128) + 1023) / 1024 * 1024;
  constexpr int W_BYTES = 9 * BLOCK_N * 128;
  const int bar_bytes = (2 * 4 + 5) * 8 + 16;
  const int room = 232448 - W_BYTES - bar_bytes;
  p.stages = std::min(4, room / p.halo_bytes);
  if (p.stages < 2) return false;
  p.base_offset_mode = mode == 2;
  p.out = cp.out; p.bias = cp.bias; p.status = cp.status;
  p.out_sn = cp.out_sn; p.out_sh = cp.out_sh; p.out_sw = cp.out_sw;
  const int smem_total = W_BYTES + p.stages * p.halo_bytes + bar_bytes;
  auto kern = conv_fwd_halo_kernel<BLOCK_N>;
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    RT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    configured[device & 63] = true;
  }
  const CUtensorMap tx = make_tmap_nhwc(a.x, a.Cin, a.W, a.H, a.N, p.PW, p.R, 1, 1);
  const CUtensorMap tw = make_tmap_2byte(a.w, (uint64_t)9 * a.Cin, a.Cout, 1, (uint64_t)9 * a.Cin, 0, 64, BLOCK_N);
  const int m_tiles = p.N * p.tiles_per_img;
  int grid = std::min(m_tiles * p.n_blocks, sm_count(device));
  grid = std::max(p.n_blocks, grid / p.n_blocks * p.n_blocks);
  kern<<<grid, CV_THREADS, smem_total, stream>>>(tx, tw, p);
  RT_LAUNCH_CHECK();
  return true;
}

}  // namespace

bool conv2d_igemm_supported(int Cin, int Cout, int KH, int KW, int stride) {
  return Cin % 64 == 0 && Cout % 8 == 0 && KH <= 7 && KW <= 7 && stride >= 1 && stride <= 4;
}

void conv2d_fwd(const Conv2dArgs& a, cudaStream_t stream) {
  check_conv(a);
  const int device = current_device();
  ConvParams p{};
  fill_common(a, p, 128);
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  p.status = status_word(device);
  static const int halo_mode = [] {
    const char* e = std::getenv("RUSTORCH_CONV_HALO");
    return e ? std::atoi(e) : 1;
  }();
  const int pad_h = a.pad_h >= 0 ? a.pad_h : a.pad;
  if (halo_mode > 0 && a.Cin == 64 && a.KH == 3 && a.KW == 3 && a.stride == 1 && a.pad == 1 && pad_h == 1 && a.out_h == 0 &&
      a.out_w == 0 && a.Cout % 64 == 0) {
    if (a.Cout % 128 == 0 ? launch_fwd_halo<128>(a, p, halo_mode, device, stream) : launch_fwd_halo<64>(a, p, halo_mode, device, stream))
      return;
  }
  if (a.Cout <= 64) launch_fwd<64>(a, p, device, stream);
  else if (a.Cout <= 128) launch_fwd<128>(a, p, device, stream);
  else launch_fwd<256>(a, p, device, stream);
}

void conv2d_wgrad(const Conv2dArgs& a, cudaStream_t stream) {
  check_conv(a);
  RT_CHECK(a.Cout % 64 == 0, "conv2d_wgrad: output channels must be a multiple of 64");
  const int device = current_device();
  ConvParams p{};
  fill_common(a, p, 64);
  p.dw = a.dw;
  p.status = status_word(device);
  static const bool three_tap = [] {
    const char* e = std::getenv("RUSTORCH_CONV_WGRAD3");
    return !(e && e[0] == '0');
  }();
  if (a.KW == 3 && three_tap) launch_wgrad3(a, p, device, stream);      // one dy fetch per kernel row
  else if (a.Cin % 128 == 0) launch_wgrad<128>(a, p, device, stream);
  else launch_wgrad<64>(a, p, device, stream);
}

}  // namespace rt
