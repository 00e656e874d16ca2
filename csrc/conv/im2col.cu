// im2col for convolutions with few input channels (the 3-channel stem of a CNN), channels-last bf16:
//
//   col[p][k] = x[n][oh * s - pad + kh][ow * s - pad + kw][c],   p = (n, oh, ow),  k = (kh * KW + kw) * Cin + c,
//   zero outside the image and for k >= KH * KW * Cin (the row is padded to k_pad, a multiple of 64).
//
// With Cin = 3 an implicit-GEMM tile cannot be fetched by TMA (a tap's channels are 6 bytes), so the patch matrix is
// written once and the convolution becomes a plain tcgen05 GEMM, col @ W^T; the weight gradient is col^T @ dy on the
// same matrix (kept for backward).  Both are bandwidth-bound on col.  A thread produces 8 consecutive k (one 16-byte
// store); the 2-byte gathers hit L1 / L2 (every input pixel is used KH * KW / s^2 times).
// Reference: src/nn/conv2d.rs im2col loops (:300-380), src/gpu/conv_ops.rs.
#include <cuda_bf16.h>

#include <algorithm>

#include "../api.h"
#include "../common/launch.h"

namespace rt {

namespace {

// A kernel row (fixed kh) of a patch is KW * C consecutive input values: x[n][ih][iw0 .. iw0 + KW - 1][0 .. C - 1] is
// contiguous in a channels-last image, so a patch is KH shifted copies of KW * C elements each; (kh, j) below walk
// them without a division per element.
__global__ void __launch_bounds__(256) im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, int N, int H,
                                                     int W, int C, int OH, int OW, int KH, int KW, int stride, int pad, int k_pad) {
  const int kv = k_pad / 8;
  const int row_len = KW * C, k_real = KH * row_len, wc = W * C;
  const long long total = (long long)N * OH * OW * kv;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    long long pix;
    int k0, ow, oh, n;
    if (total < 0x7fffffffLL) {  // 32-bit divisions: an order of magnitude cheaper than the 64-bit ones
      const unsigned tt = (unsigned)t, p32 = tt / (unsigned)kv, r32 = p32 / (unsigned)OW;
      pix = p32;
      k0 = (int)(tt - p32 * (unsigned)kv) * 8;
      ow = (int)(p32 - r32 * (unsigned)OW);
      n = (int)(r32 / (unsigned)OH);
      oh = (int)(r32 - (unsigned)n * (unsigned)OH);
    } else {
      pix = t / kv;
      k0 = (int)(t - pix * kv) * 8;
      ow = (int)(pix % OW);
      const long long r = pix / OW;
      oh = (int)(r % OH);
      n = (int)(r / OH);
    }
    const int h0 = oh * stride - pad, col0 = (ow * stride - pad) * C;       // first input row / first element of a kernel row
    int kh = k0 / row_len, j = k0 - kh * row_len;
    const __nv_bfloat16* img = x + (long long)n * H * wc;
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int ih = h0 + kh, src = col0 + j;
      const bool ok = (k0 + e < k_real) && ih >= 0 && ih < H && src >= 0 && src < wc;
      v[e] = ok ? img[(long long)ih * wc + src] : zero;
      if (++j == row_len) {
        j = 0;
        ++kh;
      }
    }
    *reinterpret_cast<uint4*>(col + pix * k_pad + k0) = *reinterpret_cast<const uint4*>(v);
  }
}

}  // namespace

void im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int stride, int pad, int k_pad,
                 cudaStream_t s) {
  RT_CHECK(k_pad % 8 == 0 && k_pad >= KH * KW * C, "im2col: padded row length must be a multiple of 8 and cover KH * KW * C");
  RT_CHECK(stride >= 1 && pad >= 0, "im2col: bad stride / padding");
  const long long work = (long long)N * OH * OW * (k_pad / 8);
  if (work == 0) return;
  const int grid = (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, 16LL * sm_count(current_device())));
  im2col_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(col), N, H, W, C, OH,
                                     OW, KH, KW, stride, pad, k_pad);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
