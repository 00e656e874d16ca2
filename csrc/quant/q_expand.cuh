// Register-level decoders of the repacked Q4_0 / Q8_0 device layout (described in q_gemv.cu), shared by the
// GEMV kernels and the dequantise-to-fp16 kernel.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

// Expand one repacked Q4_0 block (4 words) into 16 half2 of (q - 8).  Nibble pairs at bit offsets 0 and 8
// become 1024 + q (subtract 1032); pairs at offsets 4 and 12 are taken in place as 1024 + 16 q and
// mapped with one fma (x / 16 - 72), which saves their shifts: 9 instead of 12 integer/half ops per word.
__device__ __forceinline__ void expand_q4(const uint4& q, __half2 (&w)[16]) {
  const uint32_t words[4] = {q.x, q.y, q.z, q.w};
  const __half2 sub = __half2half2(__ushort_as_half(0x6408));    // 1032
  const __half2 mul = __half2half2(__ushort_as_half(0x2C00));    // 1/16
  const __half2 add = __half2half2(__ushort_as_half(0xD480));    // -72
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = words[i], hi = words[i] >> 8;
    const uint32_t b0 = (lo & 0x000F000Fu) | 0x64006400u, b1 = (lo & 0x00F000F0u) | 0x64006400u;
    const uint32_t b2 = (hi & 0x000F000Fu) | 0x64006400u, b3 = (hi & 0x00F000F0u) | 0x64006400u;
    w[i * 4 + 0] = __hsub2(*reinterpret_cast<const __half2*>(&b0), sub);
    w[i * 4 + 1] = __hfma2(*reinterpret_cast<const __half2*>(&b1), mul, add);
    w[i * 4 + 2] = __hsub2(*reinterpret_cast<const __half2*>(&b2), sub);
    w[i * 4 + 3] = __hfma2(*reinterpret_cast<const __half2*>(&b3), mul, add);
  }
}

// Streaming 16-byte load: the weights are read once per token, so they bypass L1,
// leaving it to the activations.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void expand_q8(const uint4& a, const uint4& b, __half2 (&w)[16]) {
  const uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v0 = (int)(int8_t)(words[i] & 0xFF), v1 = (int)(int8_t)((words[i] >> 8) & 0xFF);
    const int v2 = (int)(int8_t)((words[i] >> 16) & 0xFF), v3 = (int)(int8_t)(words[i] >> 24);
    w[2 * i] = __halves2half2(__int2half_rn(v0), __int2half_rn(v1));
    w[2 * i + 1] = __halves2half2(__int2half_rn(v2), __int2half_rn(v3));
  }
}

}  // namespace rt
