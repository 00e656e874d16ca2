// Dequant-fused matrix-vector products for GGUF Q4_0 / Q8_0 weights (decode path, small batch):
//
//   y[m][n] = sum_k dequant(W)[n][k] * x[m][k]  (+ bias[n]) (+ residual[m][n])      m < M <= 8 per launch
//
// The weights stay quantised in HBM (0.5625 B / weight for Q4_0) and are expanded in registers, so a
// decode step streams each weight byte exactly once.  One warp owns one output row n; lane l walks the
// 32-weight blocks l, l+32, ... of that row (coalesced 16-byte loads of the nibbles, 2-byte loads of the
// scales), multiplies them against fp16 activations read through L1, accumulates each block in half2
// and the running sum in fp32, and a warp shuffle finishes the row.
//
// Device layout ("repacked" once at load from the GGUF block stream, same information, same size):
//   Q4_0: qs [N][K/32] uint4  - word i of a block holds weights 8i..8i+7 with weight 8i+2j in bits
//                               [4j, 4j+4) and weight 8i+2j+1 in bits [16+4j, 20+4j), so that
//                               ((w >> 4j) & 0x000F000F) | 0x64006400 is the half2 (1024+q_even, 1024+q_odd)
//         d  [N][K/32] half   - block scales
//   Q8_0: qs [N][K/32][32] int8 (natural order), d as above.
// GGUF stores Q4_0 as f16 d + 16 bytes with weight j in the low and weight j+16 in the high nibble of
// byte j (block layout per the GGUF spec; the reference only records the block sizes,
// example-cli/src/model/formats/gguf.rs:131-135, and never decodes them, tensor_loader.rs:103-122).
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "q_expand.cuh"

namespace rt {

// Q8 = false: Q4_0, true: Q8_0.  M rows of x handled together (dequant shared between them).
//
// Work split: a warp owns R = 4 consecutive output rows and one of S = 4 slices of the K dimension; a CTA
// of 8 warps therefore covers 8 rows.  The four rows share every activation load (without that, each row
// re-reads x from L1 and the L1 bandwidth, not HBM, bounds the kernel), the K slices keep enough warps
// in flight when N is small, and the loads of the next step are issued before the current step is
// expanded and multiplied.  Slice sums meet in shared memory.
constexpr int QG_R = 4, QG_S = 4, QG_WARPS = 8;

template <bool Q8>
struct QRaw {
  uint4 v[Q8 ? 2 : 1];
};

template <bool Q8, int M>
__global__ void __launch_bounds__(QG_WARPS * 32) q_gemv_kernel(const void* __restrict__ qs,
                                                               const __half* __restrict__ scales,
                                                               const __half* __restrict__ x, long long ldx,
                                                               __half* __restrict__ y, long long ldy,
                                                               const __half* __restrict__ bias,
                                                               const __half* __restrict__ residual, long long ldr,
                                                               int N, int K) {
  __shared__ float part[QG_WARPS / QG_S][QG_S][QG_R][M];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / QG_S, sl = warp % QG_S;
  const int n0 = (blockIdx.x * (QG_WARPS / QG_S) + grp) * QG_R;
  const int nb = K >> 5;  // blocks per row
  const int nbs = (nb + QG_S - 1) / QG_S;
  const int b_begin = sl * nbs, b_end = min(nb, b_begin + nbs);

  long long rowoff[QG_R];  // block offset of each row (rows past N are clamped; their sums are dropped)
#pragma unroll
  for (int r = 0; r < QG_R; ++r) rowoff[r] = (long long)min(n0 + r, N - 1) * nb;

  float acc[QG_R][M];
#pragma unroll
  for (int r = 0; r < QG_R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  auto fetch = [&](int b, QRaw<Q8> (&raw)[QG_R], __half (&d)[QG_R]) {
#pragma unroll
    for (int r = 0; r < QG_R; ++r) {
      const uint4* src = reinterpret_cast<const uint4*>(qs) + (rowoff[r] + b) * (Q8 ? 2 : 1);
      raw[r].v[0] = ld_stream(src);
      if (Q8) raw[r].v[Q8 ? 1 : 0] = ld_stream(src + 1);
      d[r] = scales[rowoff[r] + b];
    }
  };

  QRaw<Q8> cur[QG_R], nxt[QG_R];
  __half dcur[QG_R], dnxt[QG_R];
  int b = b_begin + lane;
  pdl_launch_dependents();
  if (b < b_end) fetch(b, cur, dcur);   // weights do not depend on the previous kernel: in flight before the wait
  pdl_wait();
  for (; b < b_end; b += 32) {
    const bool more = b + 32 < b_end;
    if (more) fetch(b + 32, nxt, dnxt);
    __half2 w[QG_R][16];
#pragma unroll
    for (int r = 0; r < QG_R; ++r) {
      if (Q8) expand_q8(cur[r].v[0], cur[r].v[Q8 ? 1 : 0], w[r]);
      else expand_q4(cur[r].v[0], w[r]);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4* xp = reinterpret_cast<const uint4*>(x + m * ldx + (b << 5));
      __half2 xh[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(&xh[4 * i]) = __ldg(xp + i);
#pragma unroll
      for (int r = 0; r < QG_R; ++r) {
        __half2 s0 = __float2half2_rn(0.f), s1 = __float2half2_rn(0.f);
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          s0 = __hfma2(w[r][j], xh[j], s0);
          s1 = __hfma2(w[r][j + 1], xh[j + 1], s1);
        }
        const float2 f = __half22float2(__hadd2(s0, s1));
        acc[r][m] = fmaf(__half2float(dcur[r]), f.x + f.y, acc[r][m]);
      }
    }
    if (more) {
#pragma unroll
      for (int r = 0; r < QG_R; ++r) {
        cur[r] = nxt[r];
        dcur[r] = dnxt[r];
      }
    }
  }
#pragma unroll
  for (int r = 0; r < QG_R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float v = warp_sum_f(acc[r][m]);
      if (lane == 0) part[grp][sl][r][m] = v;
    }
  __syncthreads();
  // 2 groups x R rows x M activations results per CTA
  for (int i = threadIdx.x; i < (QG_WARPS / QG_S) * QG_R * M; i += blockDim.x) {
    const int g = i / (QG_R * M), r = (i / M) % QG_R, m = i % M;
    const int n = (blockIdx.x * (QG_WARPS / QG_S) + g) * QG_R + r;
    if (n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < QG_S; ++s2) v += part[g][s2][r][m];
    if (bias) v += __half2float(bias[n]);
    if (residual) v += __half2float(residual[m * ldr + n]);
    y[m * ldy + n] = __float2half(v);
  }
}

template <bool Q8>
static void launch_rows(const QGemvArgs& a, int m0, int m, cudaStream_t s) {
  const int rows_per_cta = (QG_WARPS / QG_S) * QG_R;
  const dim3 grid((a.N + rows_per_cta - 1) / rows_per_cta), block(QG_WARPS * 32);
  const __half* x = reinterpret_cast<const __half*>(a.x) + (long long)m0 * a.ldx;
  __half* y = reinterpret_cast<__half*>(a.y) + (long long)m0 * a.ldy;
  const __half* r = a.residual ? reinterpret_cast<const __half*>(a.residual) + (long long)m0 * a.ldr : nullptr;
  auto sc = reinterpret_cast<const __half*>(a.scales);
  auto bi = reinterpret_cast<const __half*>(a.bias);
#define RT_QG(MM) launch_pdl(q_gemv_kernel<Q8, MM>, grid, block, 0, s, a.qs, sc, x, a.ldx, y, a.ldy, bi, r, a.ldr, a.N, a.K)
  switch (m) {
    case 1: RT_QG(1); break;
    case 2: RT_QG(2); break;
    case 3: RT_QG(3); break;
    case 4: RT_QG(4); break;
    case 5: RT_QG(5); break;
    case 6: RT_QG(6); break;
    case 7: RT_QG(7); break;
    default: RT_QG(8); break;
  }
#undef RT_QG
  RT_LAUNCH_CHECK();
}

void q_gemv(const QGemvArgs& a, cudaStream_t stream) {
  RT_CHECK(a.K % 32 == 0, "q_gemv: K must be a multiple of 32");
  RT_CHECK(a.ldx % 8 == 0, "q_gemv: activation row stride must be a multiple of 8 halves");
  RT_CHECK((reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.qs) & 15) == 0,
           "q_gemv: x and qs must be 16-byte aligned");
  if (a.M == 0 || a.N == 0) return;
  if (a.path != 1 && q_gemv_bulk_supported(a) && (a.path == 2 || q_gemv_bulk_preferred(a))) {
    q_gemv_bulk(a, stream);
    return;
  }
  for (int m0 = 0; m0 < a.M; m0 += 8) {
    const int m = std::min(8, a.M - m0);
    if (a.q8) launch_rows<true>(a, m0, m, stream);
    else launch_rows<false>(a, m0, m, stream);
  }
}

// ---------------------------------------------------------------------------- dequantise to fp16
// Expands repacked weights to a dense fp16 [N][K] matrix: the prefill / large-batch path, where the matrix
// then feeds the tcgen05 GEMM (the expansion is one pass over 0.56 + 2 bytes per weight, small against a
// GEMM over hundreds of rows).
template <bool Q8>
__global__ void __launch_bounds__(256) dequant_f16_kernel(const void* __restrict__ qs,
                                                          const __half* __restrict__ scales,
                                                          __half* __restrict__ out, long long n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  __half2 w[16];
  const uint4* src = reinterpret_cast<const uint4*>(qs) + i * (Q8 ? 2 : 1);
  if (Q8) expand_q8(ld_stream(src), ld_stream(src + (Q8 ? 1 : 0)), w);
  else expand_q4(ld_stream(src), w);
  const __half2 d = __half2half2(scales[i]);
  uint4* dst = reinterpret_cast<uint4*>(out + i * 32);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    __half2 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __hmul2(w[q * 4 + j], d);
    dst[q] = *reinterpret_cast<const uint4*>(v);
  }
}

void dequant_f16(const void* qs, const void* scales, void* out, long long n_blocks, bool q8, cudaStream_t s) {
  if (n_blocks == 0) return;
  const unsigned grid = (unsigned)((n_blocks + 255) / 256);
  if (q8) dequant_f16_kernel<true><<<grid, 256, 0, s>>>(qs, reinterpret_cast<const __half*>(scales),
                                                      reinterpret_cast<__half*>(out), n_blocks);
  else dequant_f16_kernel<false><<<grid, 256, 0, s>>>(qs, reinterpret_cast<const __half*>(scales),
                                                      reinterpret_cast<__half*>(out), n_blocks);
  RT_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------- repack
// GGUF Q4_0 block stream [rows][K/32][18] -> qs (uint4 per block, layout above) + scales.
__global__ void repack_q4_0_kernel(const uint8_t* __restrict__ blocks, uint4* __restrict__ qs,
                                   __half* __restrict__ scales, long long n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  const uint8_t* b = blocks + i * 18;
  scales[i] = __ushort_as_half((unsigned short)(b[0] | (b[1] << 8)));
  uint32_t out[4];
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int k = wi * 8 + e;  // weight index in the block
      const uint32_t q = (k < 16) ? (b[2 + k] & 0x0F) : (b[2 + k - 16] >> 4);
      const int shift = (e & 1) ? 16 + 4 * (e >> 1) : 4 * (e >> 1);
      word |= q << shift;
    }
    out[wi] = word;
  }
  qs[i] = make_uint4(out[0], out[1], out[2], out[3]);
}

// GGUF Q8_0 block stream [rows][K/32][34] -> qs int8 [.][32] + scales.
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ blocks, int8_t* __restrict__ qs,
                                   __half* __restrict__ scales, long long n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks) return;
  const uint8_t* b = blocks + i * 34;
  scales[i] = __ushort_as_half((unsigned short)(b[0] | (b[1] << 8)));
  for (int k = 0; k < 32; ++k) qs[i * 32 + k] = (int8_t)b[2 + k];
}

void repack_q4_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s) {
  if (n_blocks == 0) return;
  repack_q4_0_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const uint8_t*>(blocks), reinterpret_cast<uint4*>(qs), reinterpret_cast<__half*>(scales), n_blocks);
  RT_LAUNCH_CHECK();
}

void repack_q8_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s) {
  if (n_blocks == 0) return;
  repack_q8_0_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const uint8_t*>(blocks), reinterpret_cast<int8_t*>(qs), reinterpret_cast<__half*>(scales), n_blocks);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
