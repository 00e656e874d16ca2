// Shared pieces of the tcgen05 flash-attention kernels (forward, dK/dV, dQ).
//
// Geometry common to all three kernels: 128 query rows x 128 key rows per tile; one thread
// owns one row of the 128x128 score tile because tcgen05.ld.32x32b hands TMEM lane i to
// thread i of the 4 "row" warps, so row max / row sum need no shuffles.  Probabilities
// (and dS) are staged in shared memory as a [128 rows][128 cols] bf16 tile made of two
// 64-column halves, each half with 128-byte rows under the 128B swizzle.  That single
// layout is at once
//   * a K-major  A operand  (M = rows, K = cols)  for  P @ V   and  dS @ K
//   * an MN-major A operand (M = cols, K = rows)  for  P^T @ dO and  dS^T @ Q
// so no transposed copy of P or dS is ever made.
#pragma once
#include "../common/ptx.cuh"

namespace rt {

constexpr int ATT_BM = 128;  // query rows per tile
constexpr int ATT_BN = 128;  // key rows per tile
constexpr int ATT_HALF_BYTES = 128 * 128;  // one 64-column half: 128 rows x 128 B

// Store 32 consecutive columns [col0, col0+32) of row `row` (fp32 -> bf16, or fp16 with F16) into the swizzled
// [128][128] 16-bit staging tile at `tile`.
template <bool F16 = false>
__device__ __forceinline__ void stage_row_chunk_bf16(uint8_t* tile, int row, int col0,
                                                     const float (&v)[32]) {
  const int half = col0 >> 6;
  const int c16_0 = (col0 & 63) >> 3;  // first 16-byte chunk index inside the 128 B row
  uint8_t* rowp = tile + half * ATT_HALF_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w;
    w.x = pack_2x16<F16>(v[q * 8 + 0], v[q * 8 + 1]);
    w.y = pack_2x16<F16>(v[q * 8 + 2], v[q * 8 + 3]);
    w.z = pack_2x16<F16>(v[q * 8 + 4], v[q * 8 + 5]);
    w.w = pack_2x16<F16>(v[q * 8 + 6], v[q * 8 + 7]);
    const int c16 = (c16_0 + q) ^ (row & 7);
    *reinterpret_cast<uint4*>(rowp + c16 * 16) = w;
  }
}

// Descriptors for the staging tile above.
// As K-major A operand, k-step kk (16 columns each, kk in [0,8)).
__device__ __forceinline__ uint64_t stage_desc_kmajor(uint32_t tile_addr, int kk) {
  return make_smem_desc_sw128(tile_addr + (kk >> 2) * ATT_HALF_BYTES + (kk & 3) * 32, 16, 1024);
}
// As MN-major A operand (M = the 128 columns, K = rows), k-step kk (16 rows each).
__device__ __forceinline__ uint64_t stage_desc_mnmajor(uint32_t tile_addr, int kk) {
  return make_smem_desc_sw128(tile_addr + kk * 2048, ATT_HALF_BYTES, 1024);
}

// A [128 rows][D] bf16 tile loaded by TMA as D/64 column halves of 128-byte rows.
// K-major use (reduction over D): k-step kk covers 16 of the D columns.
template <int D>
__device__ __forceinline__ uint64_t tile_desc_kmajor(uint32_t tile_addr, int kk) {
  return make_smem_desc_sw128(tile_addr + (kk >> 2) * ATT_HALF_BYTES + (kk & 3) * 32, 16, 1024);
}
// MN-major use (N or M = D, reduction over the 128 rows): k-step kk covers 16 rows.
template <int D>
__device__ __forceinline__ uint64_t tile_desc_mnmajor(uint32_t tile_addr, int kk) {
  return make_smem_desc_sw128(tile_addr + kk * 2048, ATT_HALF_BYTES, 1024);
}

// Issue the TMA loads for one [128][D] tile of a [B][T][H][D]-strided tensor.
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar,
                                          int row0, int head, int batch) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c)
    tma_load_4d(dst + c * ATT_HALF_BYTES, tmap, bar, c * 64, row0, head, batch);
}

}  // namespace rt
