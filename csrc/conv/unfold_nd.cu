// Patch gather / scatter for convolutions of one to three spatial dimensions with stride, padding, dilation and
// groups, on channels-last bf16 tensors x[N][D][H][W][C] (1-D and 2-D convolutions use D = 1 / D = H = 1):
//
//   unfold_nd : col[g][m][tap * Cg + c] = x[n][od*sd - pd + kd*dd][oh*sh - ph + kh*dh][ow*sw - pw + kw*dw][g*Cg + c]
//               (zero outside the image), m = ((n*OD + od)*OH + oh)*OW + ow, rows padded with zeros to k_pad columns
//   fold_nd   : x[n][d][h][w][g*Cg + c] = sum over the taps and output positions that read this pixel of col[g][m][...]
//               (a gather over at most KD*KH*KW taps per element: no atomics, every element written exactly once)
//
// The convolution itself is then one tcgen05 GEMM per group over the patch matrix (batched over groups), its weight
// gradient a GEMM with both operands transposed, and its input gradient (also the forward pass of a transposed
// convolution) a GEMM followed by fold_nd.  The reference's conv3d kernel walks the same index space with one
// thread per output element and a scalar inner product (src/gpu/cuda_kernels.cu:133-198; layer arithmetic in
// src/nn/conv3d.rs:74-237, src/nn/conv_transpose_3d.rs).
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

struct UnfoldGeom {
  int N, D, H, W, C;      // input, channels-last
  int OD, OH, OW;         // output positions
  int KD, KH, KW;
  int sd, sh, sw, pd, ph, pw, dd, dh, dw;
  int groups, Cg;         // Cg = C / groups
  int k_pad;              // row length of col (>= KD*KH*KW*Cg), multiple of 8
};

template <int VEC>  // channels per thread: 8 (16-byte accesses) or 1
__global__ void __launch_bounds__(256) unfold_nd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col,
                                                        const UnfoldGeom g, long long M, long long x_elems, long long col_elems,
                                                        int* status) {
  const int taps = g.KD * g.KH * g.KW;
  const int cv = g.Cg / VEC;                       // vectors per tap
  const long long per_row = (long long)taps * cv;
  const long long total = (long long)g.groups * M * per_row;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int v = int(t % cv);
    long long r = t / cv;
    const int tap = int(r % taps);
    r /= taps;
    const long long m = r % M;
    const int grp = int(r / M);
    const int kw = tap % g.KW, kh = (tap / g.KW) % g.KH, kd = tap / (g.KW * g.KH);
    long long q = m;
    const int ow = int(q % g.OW); q /= g.OW;
    const int oh = int(q % g.OH); q /= g.OH;
    const int od = int(q % g.OD);
    const int n = int(q / g.OD);
    const int id = od * g.sd - g.pd + kd * g.dd, ih = oh * g.sh - g.ph + kh * g.dh, iw = ow * g.sw - g.pw + kw * g.dw;
    const bool in = id >= 0 && id < g.D && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
    __nv_bfloat16* dst = col + ((long long)grp * M + m) * g.k_pad + (long long)tap * g.Cg + v * VEC;
    const __nv_bfloat16* src = x + ((((long long)n * g.D + id) * g.H + ih) * g.W + iw) * g.C + grp * g.Cg + v * VEC;
    // checked builds: both addresses against the tensors' element counts
    if (!RT_GUARD((dst - col) + VEC - 1, col_elems, status) || (in && !RT_GUARD((src - x) + VEC - 1, x_elems, status))) continue;
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(dst) = in ? *reinterpret_cast<const uint4*>(src) : make_uint4(0u, 0u, 0u, 0u);
    } else {
      *dst = in ? *src : __float2bfloat16(0.f);
    }
  }
  // zero the padding columns [taps * Cg, k_pad) of every row
  const int pad = g.k_pad - taps * g.Cg;
  if (pad > 0) {
    const long long rows = (long long)g.groups * M;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < rows * pad; t += (long long)gridDim.x * blockDim.x) {
      const long long at = (t / pad) * g.k_pad + taps * g.Cg + (t % pad);
      if (RT_GUARD(at, col_elems, status)) col[at] = __float2bfloat16(0.f);
    }
  }
}

__global__ void __launch_bounds__(256) fold_nd_kernel(const __nv_bfloat16* __restrict__ col, __nv_bfloat16* __restrict__ x,
                                                      const UnfoldGeom g, long long M, long long col_elems, int* status) {
  const long long total = (long long)g.N * g.D * g.H * g.W * g.C;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int c = int(t % g.C);
    long long q = t / g.C;
    const int iw = int(q % g.W); q /= g.W;
    const int ih = int(q % g.H); q /= g.H;
    const int id = int(q % g.D);
    const int n = int(q / g.D);
    const int grp = c / g.Cg, cc = c - grp * g.Cg;
    float acc = 0.f;
    for (int kd = 0; kd < g.KD; ++kd) {
      const int nd = id + g.pd - kd * g.dd;
      if (nd < 0 || nd % g.sd) continue;
      const int od = nd / g.sd;
      if (od >= g.OD) continue;
      for (int kh = 0; kh < g.KH; ++kh) {
        const int nh = ih + g.ph - kh * g.dh;
        if (nh < 0 || nh % g.sh) continue;
        const int oh = nh / g.sh;
        if (oh >= g.OH) continue;
        for (int kw = 0; kw < g.KW; ++kw) {
          const int nw = iw + g.pw - kw * g.dw;
          if (nw < 0 || nw % g.sw) continue;
          const int ow = nw / g.sw;
          if (ow >= g.OW) continue;
          const long long m = (((long long)n * g.OD + od) * g.OH + oh) * g.OW + ow;
          const int tap = (kd * g.KH + kh) * g.KW + kw;
          const long long at = ((long long)grp * M + m) * g.k_pad + (long long)tap * g.Cg + cc;
          if (RT_GUARD(at, col_elems, status)) acc += __bfloat162float(col[at]);
        }
      }
    }
    x[t] = __float2bfloat16(acc);
  }
}

UnfoldGeom geom_of(const UnfoldArgs& a) {
  UnfoldGeom g{};
  g.N = a.N; g.D = a.D; g.H = a.H; g.W = a.W; g.C = a.C;
  g.OD = a.OD; g.OH = a.OH; g.OW = a.OW;
  g.KD = a.KD; g.KH = a.KH; g.KW = a.KW;
  g.sd = a.stride[0]; g.sh = a.stride[1]; g.sw = a.stride[2];
  g.pd = a.pad[0]; g.ph = a.pad[1]; g.pw = a.pad[2];
  g.dd = a.dilation[0]; g.dh = a.dilation[1]; g.dw = a.dilation[2];
  g.groups = a.groups;
  g.Cg = a.C / a.groups;
  g.k_pad = a.k_pad;
  return g;
}

void check(const UnfoldArgs& a) {
  RT_CHECK(a.groups >= 1 && a.C % a.groups == 0, "unfold_nd: channels must divide into the groups");
  RT_CHECK(a.k_pad % 8 == 0 && a.k_pad >= a.KD * a.KH * a.KW * (a.C / a.groups), "unfold_nd: k_pad must be a multiple of 8 that holds a patch");
  for (int i = 0; i < 3; ++i) RT_CHECK(a.stride[i] >= 1 && a.dilation[i] >= 1 && a.pad[i] >= 0, "unfold_nd: bad stride / dilation / padding");
}

}  // namespace

void unfold_nd(const UnfoldArgs& a, cudaStream_t s) {
  check(a);
  const UnfoldGeom g = geom_of(a);
  const long long M = (long long)a.N * a.OD * a.OH * a.OW;
  if (M == 0) return;
  const int taps = a.KD * a.KH * a.KW;
  const bool vec = (g.Cg % 8 == 0) && (a.C % 8 == 0);
  const long long work = (long long)a.groups * M * taps * (vec ? g.Cg / 8 : g.Cg);
  const int grid = (int)std::min<long long>((work + 255) / 256, 32LL * sm_count(current_device()));
  auto* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  auto* col = reinterpret_cast<__nv_bfloat16*>(a.col);
  const long long x_elems = (long long)a.N * a.D * a.H * a.W * a.C, col_elems = (long long)a.groups * M * a.k_pad;
  int* status = status_word(current_device());
  if (vec) unfold_nd_kernel<8><<<std::max(grid, 1), 256, 0, s>>>(x, col, g, M, x_elems, col_elems, status);
  else unfold_nd_kernel<1><<<std::max(grid, 1), 256, 0, s>>>(x, col, g, M, x_elems, col_elems, status);
  RT_LAUNCH_CHECK();
}

void fold_nd(const UnfoldArgs& a, cudaStream_t s) {
  check(a);
  const UnfoldGeom g = geom_of(a);
  const long long M = (long long)a.N * a.OD * a.OH * a.OW;
  const long long total = (long long)a.N * a.D * a.H * a.W * a.C;
  if (total == 0) return;
  const int grid = (int)std::min<long long>((total + 255) / 256, 32LL * sm_count(current_device()));
  fold_nd_kernel<<<std::max(grid, 1), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(a.col), reinterpret_cast<__nv_bfloat16*>(a.x), g, M,
                                                   (long long)a.groups * M * a.k_pad, status_word(current_device()));
  RT_LAUNCH_CHECK();
}

}  // namespace rt
