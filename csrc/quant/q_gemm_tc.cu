// Dequant-fused tensor-core GEMM for GGUF Q4_0 / Q8_0 weights (batched decode and short prefill, 8 < M <= 256):
//
//   y[m][n] = sum_k dequant(W)[n][k] * x[m][k]  (+ bias[n]) (+ residual[m][n])        x, y fp16
//
// The weights stay quantised in HBM and are read exactly once per call, whatever M is: a CTA owns 128 weight rows
// (the M side of the MMA) and a slice of K; the activations are the N side (M padded to 16 / 32 / 64 / 128 / 256).
//
//   warp 0       producer of raw nibbles / bytes: TMA tiles of 128 rows x 128 B, 128-byte swizzle so that the row-per-
//                thread reads below are bank-conflict free
//   warp 10      producer of the SW128 K-major tiles of x (64 k x M_pad rows)
//   warp 1       tcgen05.mma issuer, accumulator D[128 weight rows][M_pad] fp32 in TMEM
//   warps 2..9   dequantise: thread (row r, half hb) expands one 32-weight block per 64-k step to fp16 * scale and
//                stores it as four 16-byte chunks of row r of the A tile in the canonical SW128 K-major layout
//                (chunk ^ (r & 7)), then fence.proxy.async + mbarrier arrive; afterwards the same warps are the
//                epilogue (TMEM quarter = warp & 3, column half = (warp - 2) >> 2)
//
// Split-K: grid.y CTAs share an output tile; each writes its fp32 partial to scratch and the last to arrive (counter
// per tile, reset by that CTA) sums them in split order, adds bias / residual and writes fp16.  No second kernel.
// Block scales are read straight from global memory one raw stage ahead (their row pitch, K/32 * 2 bytes, need not
// be a multiple of 16, which a tensor map would require; tensor-parallel shards have such K).
// All waits are bounded; on expiry the CTA raises its abort flag, lets copies land, frees TMEM and leaves.
//
// GGUF block formats per the GGUF spec; the reference only records block sizes and never decodes them
// (example-cli/src/model/formats/gguf.rs:131-135, tensor_loader.rs:103-122).
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "q_expand.cuh"

namespace rt {

namespace {

constexpr int QT_THREADS = 352;   // warp 0 raw producer, 1 MMA, 2..9 dequantise + epilogue, 10 activation producer
constexpr int QT_X_WARP = 10;
constexpr int QT_DQ_WARPS = 8;
constexpr int QT_RAW_STAGES = 3;   // most; small activation tiles use 2 so that two CTAs share an SM
constexpr int QT_MAX_SLOTS = 6;
constexpr int QT_RAW_BYTES = 128 * 128;   // 128 rows x 128 B
constexpr int QT_ATOM_BYTES = 128 * 128;  // one SW128 atom: 128 rows x 64 halves
constexpr int QT_A_BYTES = 2 * QT_ATOM_BYTES;   // an operand slot holds two atoms (128 k): one handshake per 128 k

struct QtParams {
  const __half* scales;
  __half* y;
  const __half* bias;
  const __half* residual;
  float* partial;        // [tiles][splits][m_pad][128]
  int* counters;         // [tiles], zero between calls
  long long ldy, ldr;
  int M, N, K, m_pad, op_slots, raw_stages, chunks_per_split, total_chunks;
  int* status;
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Position in a ring of n slots and the parity of the current pass over it.
struct Ring {
  int i, n;
  uint32_t ph;
  __device__ __forceinline__ Ring(int n_) : i(0), n(n_), ph(0) {}
  __device__ __forceinline__ void next() {
    if (++i == n) {
      i = 0;
      ph ^= 1;
    }
  }
};

__device__ __forceinline__ uint4 pack8(const __half2 (&w)[16], int i) {
  uint4 v;
  v.x = *reinterpret_cast<const uint32_t*>(&w[i]);
  v.y = *reinterpret_cast<const uint32_t*>(&w[i + 1]);
  v.z = *reinterpret_cast<const uint32_t*>(&w[i + 2]);
  v.w = *reinterpret_cast<const uint32_t*>(&w[i + 3]);
  return v;
}

template <bool Q8>
__global__ void __launch_bounds__(QT_THREADS, 2) q_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_raw,
                                                                  const __grid_constant__ CUtensorMap tm_x, const QtParams p) {
  constexpr int KRAW = Q8 ? 128 : 256;   // k covered by one raw stage (128 B per row)
  constexpr int SUBS = KRAW / 64;        // 64-k atoms per raw stage
  constexpr int STEPS = KRAW / 128;      // 128-k operand slots per raw stage
  // The swizzled tiles need a 1024-byte aligned base.  Dynamic shared memory starts right after the 1 KB the driver
  // keeps per block, so it is aligned; the launch reserves no slack (two CTAs must fit one SM), and a base that is
  // not aligned ends the kernel with an error code before anything is touched.
  extern __shared__ __align__(1024) uint8_t qt_smem_raw[];
  uint8_t* smem = qt_smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, RT_ERR_BOUNDS);
    return;
  }
  const int OS = p.op_slots, MP = p.m_pad, RS = p.raw_stages;
  const int x_atom = MP * 128;            // one 64-k activation box
  const int x_bytes = 2 * x_atom;
  uint8_t* raw = smem;
  uint8_t* a_t = raw + RS * QT_RAW_BYTES;
  uint8_t* x_t = a_t + OS * QT_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(x_t + OS * x_bytes);
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + QT_RAW_STAGES;
  uint64_t* x_full = raw_empty + QT_RAW_STAGES;
  uint64_t* a_full = x_full + QT_MAX_SLOTS;
  uint64_t* op_empty = a_full + QT_MAX_SLOTS;
  uint64_t* acc_full = op_empty + QT_MAX_SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(tmem_slot + 1);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int n0 = tile * 128;
  const int c_begin = split * p.chunks_per_split;
  const int c_end = min(p.total_chunks, c_begin + p.chunks_per_split);
  const int nb = p.K >> 5;
  const uint32_t tmem_cols = MP < 32 ? 32u : (uint32_t)MP;

  if (threadIdx.x == 0) {
    for (int i = 0; i < QT_RAW_STAGES; ++i) {
      mbar_init(&raw_full[i], 1);
      mbar_init(&raw_empty[i], QT_DQ_WARPS);
    }
    for (int i = 0; i < QT_MAX_SLOTS; ++i) {
      mbar_init(&x_full[i], 1);
      mbar_init(&a_full[i], QT_DQ_WARPS);
      mbar_init(&op_empty[i], 1);
    }
    mbar_init(acc_full, 1);
    ctl->abort = 0;
    *last_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_raw);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  const uint32_t tmem_base = *tmem_slot;
  auto steps_of = [&](int c) { return min(STEPS, (p.K - c * KRAW + 127) >> 7); };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    // Raw weight tiles: up to raw_stages chunks ahead of the dequantisers (blocking waits: the thread sleeps in hardware).
    if (lane == 0) {
      Ring rr(RS);
      for (int c = c_begin; c < c_end; ++c) {
        if (!mbar_wait(&raw_empty[rr.i], rr.ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(&raw_full[rr.i], QT_RAW_BYTES);
        tma_load_2d(raw + rr.i * QT_RAW_BYTES, &tm_raw, &raw_full[rr.i], c * 32, n0);
        rr.next();
      }
    }
  } else if (warp == QT_X_WARP) {
    // Activation tiles: up to op_slots steps ahead of the MMAs.  A warp of its own, so that neither producer holds
    // up the other and neither has to poll.
    if (lane == 0) {
      Ring xr(OS);
      bool ok = true;
      pdl_wait();                       // the activations come from the previous kernel; the weights above do not
      for (int c = c_begin; c < c_end && ok; ++c) {
        const int ns = steps_of(c);
        for (int st = 0; st < ns; ++st) {
          if (!mbar_wait(&op_empty[xr.i], xr.ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&x_full[xr.i], x_bytes);
          const int k0 = c * KRAW + st * 128;      // the second box may lie past K: it reads as zeros
          tma_load_3d(x_t + xr.i * x_bytes, &tm_x, &x_full[xr.i], k0, 0, 0);
          tma_load_3d(x_t + xr.i * x_bytes + x_atom, &tm_x, &x_full[xr.i], k0 + 64, 0, 0);
          xr.next();
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(128, MP, false, false, false);
      Ring r(OS);
      bool first = true, ok = true;
      for (int c = c_begin; c < c_end && ok; ++c) {
        const int ns = steps_of(c);
        for (int st = 0; st < ns; ++st) {
          const int j = r.i;
          if (!mbar_wait(&x_full[j], r.ph, ctl, p.status, RT_ERR_TIMEOUT_MMA) ||
              !mbar_wait(&a_full[j], r.ph, ctl, p.status, RT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(a_t + j * QT_A_BYTES), sb = smem_u32(x_t + j * x_bytes);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t oa = (kk >> 2) * QT_ATOM_BYTES + (kk & 3) * 32, ob = (kk >> 2) * x_atom + (kk & 3) * 32;
            umma_f16_ss(tmem_base, make_smem_desc_sw128(sa + oa, 16, 1024), make_smem_desc_sw128(sb + ob, 16, 1024), idesc,
                        (!first || kk > 0) ? 1u : 0u);
          }
          first = false;
          umma_commit(&op_empty[j]);
          r.next();
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------- dequantise, then epilogue
    const int t = threadIdx.x - 64;
    const int r = t & 127, hb = t >> 7;
    const int n = n0 + r;
    const bool row_ok = n < p.N;
    const __half* srow = p.scales + (long long)min(n, p.N - 1) * nb;
    // Scales of a row's chunk are SPC consecutive halves (16 B for Q4_0, 8 B for Q8_0): one vector load when the row
    // pitch keeps them aligned and the chunk lies inside the row, else one 2-byte load per block.
    constexpr int SPC = KRAW / 32;
    const bool vec_scales = (nb % SPC) == 0;
    auto load_scales = [&](int c, __half (&d)[SUBS]) {
      const bool live = row_ok && c < c_end;
      if (vec_scales) {
        __half tmp[SPC];
        if (live) {
          if (SPC == 8) *reinterpret_cast<uint4*>(tmp) = __ldg(reinterpret_cast<const uint4*>(srow + (long long)c * SPC));
          else *reinterpret_cast<uint2*>(tmp) = __ldg(reinterpret_cast<const uint2*>(srow + (long long)c * SPC));
        }
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub) d[sub] = live ? (hb ? tmp[sub * 2 + 1] : tmp[sub * 2]) : __ushort_as_half(0);
      } else {
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub) {
          const int b = c * SPC + sub * 2 + hb;
          d[sub] = (live && b < nb) ? srow[b] : __ushort_as_half(0);
        }
      }
    };
    __half dcur[SUBS], dnxt[SUBS];
    load_scales(c_begin, dcur);
    Ring rr(RS), orr(OS);
    bool ok = true;
    for (int c = c_begin; c < c_end && ok; ++c) {
      const int s = rr.i;
      load_scales(c + 1, dnxt);
      if (!mbar_wait(&raw_full[s], rr.ph, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) break;
      const uint8_t* rrow = raw + s * QT_RAW_BYTES + r * 128;
      const int ns = steps_of(c);
#pragma unroll
      for (int st = 0; st < STEPS; ++st) {
        if (st >= ns) break;
        const int j = orr.i;
        uint8_t* arow = a_t + j * QT_A_BYTES + r * 128;
#pragma unroll
        for (int half_step = 0; half_step < 2; ++half_step) {
          const int sub = st * 2 + half_step;
          __half2 w[16];
          if (Q8) {
            const int cj = (sub * 2 + hb) * 2;
            const uint4 q0 = *reinterpret_cast<const uint4*>(rrow + ((cj ^ (r & 7)) << 4));
            const uint4 q1 = *reinterpret_cast<const uint4*>(rrow + (((cj + 1) ^ (r & 7)) << 4));
            expand_q8(q0, q1, w);
          } else {
            const int cj = sub * 2 + hb;
            const uint4 q = *reinterpret_cast<const uint4*>(rrow + ((cj ^ (r & 7)) << 4));
            expand_q4(q, w);
          }
          const __half2 d2 = __half2half2(dcur[sub]);
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = __hmul2(w[i], d2);
          if (half_step == 0 && !mbar_wait(&op_empty[j], orr.ph ^ 1, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
            ok = false;
            break;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e)
            *reinterpret_cast<uint4*>(arow + half_step * QT_ATOM_BYTES + (((hb * 4 + e) ^ (r & 7)) << 4)) = pack8(w, e * 4);
        }
        if (!ok) break;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[j]);
        orr.next();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[s]);
      rr.next();
#pragma unroll
      for (int sub = 0; sub < SUBS; ++sub) dcur[sub] = dnxt[sub];
    }
    pdl_wait();                          // residual / y / split-K scratch: only after the previous kernel has finished
    // ---- epilogue: D[lane = weight row][col = activation row]
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const int nl = quarter * 32 + lane;            // row of the tile this thread reads from TMEM
    const int ne = n0 + nl;
    const int groups = MP / 16;                    // 16-column groups; halves of them per warp
    const int g_begin = col_half * ((groups + 1) / 2), g_end = min(groups, g_begin + (groups + 1) / 2);
    if (ok && mbar_wait(acc_full, 0, ctl, p.status, RT_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      float* mypart = p.partial + ((long long)tile * splits + split) * MP * 128;
      for (int g = g_begin; g < g_end; ++g) {
        uint32_t v[16];
        __syncwarp();
        tmem_ld_32x32b_x16(tmem_base + (uint32_t(quarter * 32) << 16) + g * 16, v);
        tmem_ld_wait();
        if (splits > 1) {
#pragma unroll
          for (int i = 0; i < 16; ++i) mypart[(g * 16 + i) * 128 + nl] = __uint_as_float(v[i]);
        } else if (ne < p.N) {
          const float bv = p.bias ? __half2float(p.bias[ne]) : 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = g * 16 + i;
            if (m < p.M) {
              float o = __uint_as_float(v[i]) + bv;
              if (p.residual) o += __half2float(p.residual[m * p.ldr + ne]);
              p.y[m * p.ldy + ne] = __float2half(o);
            }
          }
        }
      }
      tc_fence_before();
    }
    if (splits > 1) {
      // the last CTA of this tile to get here reduces all partials (named barrier over the 8 epilogue warps)
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (t == 0) {
        const int prev = atomicAdd(p.counters + tile, 1);
        *last_flag = (prev == splits - 1) ? 1 : 0;
        if (prev == splits - 1) p.counters[tile] = 0;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*last_flag && !ctl->abort) {
        __threadfence();
        const float* base = p.partial + (long long)tile * splits * MP * 128;
        // thread t: column nl2 = t & 127, activation rows m = (t >> 7), +2, ...
        const int nl2 = t & 127, ne2 = n0 + nl2;
        if (ne2 < p.N) {
          const float bv = p.bias ? __half2float(p.bias[ne2]) : 0.f;
          for (int m = t >> 7; m < p.M; m += 2) {
            float o = bv;
            for (int sp = 0; sp < splits; ++sp) o += __ldcg(base + ((long long)sp * MP + m) * 128 + nl2);
            if (p.residual) o += __half2float(p.residual[m * p.ldr + ne2]);
            p.y[m * p.ldy + ne2] = __float2half(o);
          }
        }
      }
    }
  }

  // Common exit: on abort give in-flight bulk copies time to land, then release TMEM.
  __syncwarp();
  if (ctl->abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

int pad_m(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

}  // namespace

bool q_gemm_tc_supported(int M, int N, int K) { return M >= 1 && M <= 256 && N >= 1 && K >= 32 && K % 32 == 0; }

// Scratch: fp32 words for the split-K partials, and one int32 counter per 128-row tile (zeroed once by the caller).
void q_gemm_tc_scratch(int M, int N, int K, bool q8, int sms, long long* partial_floats, int* counters, int* splits_out) {
  const int kraw = q8 ? 128 : 256;
  const int total = (K + kraw - 1) / kraw, tiles = (N + 127) / 128;
  // CTAs run one per SM: cost = waves x (chunks per CTA + fixed part); pick the cheapest split count.
  int splits = 1;
  double best = 1e30;
  // Cost of a split count: the busiest SM gets n = ceil(CTAs / SMs) CTAs of (chunks + fixed part) each.  Up to 32 rows
  // two CTAs share an SM; measured, a co-resident pair finishes in ~1.43x the time of one CTA (they hide each
  // other's latencies but share the issue slots), so n CTAs cost (n / 2) * 1.43 + (n % 2).
  const bool pairs = pad_m(M) <= 32;
  for (int s = 1; s <= std::min(16, std::max(1, total / 2)); ++s) {
    const int per_s = (total + s - 1) / s, n = (tiles * s + sms - 1) / sms;
    const double rounds = pairs ? (n / 2) * 1.43 + (n % 2) : (double)n;
    const double cost = rounds * (per_s + 1.5);
    if (cost < best - 1e-9) best = cost, splits = s;
  }
  const int per = (total + splits - 1) / splits;
  splits = (total + per - 1) / per;
  *partial_floats = splits > 1 ? (long long)tiles * splits * pad_m(M) * 128 : 0;
  *counters = tiles;
  *splits_out = splits;
}

void q_gemm_tc(const QGemvArgs& a, void* partial, int* counters, cudaStream_t stream) {
  RT_CHECK(q_gemm_tc_supported(a.M, a.N, a.K), "q_gemm_tc: needs 1 <= M <= 256 and K a multiple of 32");
  RT_CHECK(a.ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0, "q_gemm_tc: activations must be 16-byte aligned rows");
  const int device = current_device();
  const int kraw = a.q8 ? 128 : 256;
  QtParams p{};
  p.scales = reinterpret_cast<const __half*>(a.scales);
  p.y = reinterpret_cast<__half*>(a.y);
  p.bias = reinterpret_cast<const __half*>(a.bias);
  p.residual = reinterpret_cast<const __half*>(a.residual);
  p.ldy = a.ldy; p.ldr = a.ldr;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.m_pad = pad_m(a.M);
  p.op_slots = 2;                                       // 128 k each
  // <= 32 rows: two CTAs per SM (113 KB each); 256 rows: the activation slots take 128 KB
  p.raw_stages = (p.m_pad <= 32 || p.m_pad == 256) ? 2 : QT_RAW_STAGES;
  long long pf; int nc, splits;
  q_gemm_tc_scratch(a.M, a.N, a.K, a.q8, sm_count(device), &pf, &nc, &splits);
  p.total_chunks = (a.K + kraw - 1) / kraw;
  p.chunks_per_split = (p.total_chunks + splits - 1) / splits;
  RT_CHECK(splits == 1 || (partial != nullptr && counters != nullptr), "q_gemm_tc: split-K scratch missing");
  p.partial = reinterpret_cast<float*>(partial);
  p.counters = counters;
  p.status = status_word(device);
  const uint64_t row_bytes = (uint64_t)(a.K / 32) * (a.q8 ? 32 : 16);
  const CUtensorMap tr = make_tmap_words_sw128(a.qs, row_bytes, a.N, 128);
  const CUtensorMap tx = make_tmap_2byte(a.x, a.K, a.M, 1, a.ldx, 0, 64, p.m_pad);
  const int smem = p.raw_stages * QT_RAW_BYTES + p.op_slots * (QT_A_BYTES + 2 * p.m_pad * 128) + 512;
  RT_CHECK(smem <= 227 * 1024, "q_gemm_tc: shared-memory budget exceeded");
  const dim3 grid((a.N + 127) / 128, splits);
  if (a.q8) {
    static bool cfg[64] = {false};
    if (!cfg[device]) {
      RT_CUDA_CHECK(cudaFuncSetAttribute(q_gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      cfg[device] = true;
    }
    launch_pdl(q_gemm_tc_kernel<true>, grid, dim3(QT_THREADS), (size_t)smem, stream, tr, tx, p);
  } else {
    static bool cfg[64] = {false};
    if (!cfg[device]) {
      RT_CUDA_CHECK(cudaFuncSetAttribute(q_gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      cfg[device] = true;
    }
    launch_pdl(q_gemm_tc_kernel<false>, grid, dim3(QT_THREADS), (size_t)smem, stream, tr, tx, p);
  }
  RT_LAUNCH_CHECK();
}

}  // namespace rt
