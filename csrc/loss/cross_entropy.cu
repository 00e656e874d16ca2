// Fused softmax cross-entropy over bf16 logits: one pass computes the per-row loss and
// overwrites the logits in place with d(loss)/d(logits) = (softmax - onehot) * grad_scale,
// so the [tokens x vocab] probabilities never exist as a separate tensor.  The row is staged
// in shared memory when it fits (one HBM read + one write per logit).
// Columns >= vocab (padding added so rows are 16-byte aligned) are excluded and get zero
// gradient.  The reference's CrossEntropyLoss recurses forever
// (src/nn/loss.rs:58-69,98-106); semantics here are the standard mean-reduced NLL of softmax.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

template <bool STAGED>
__global__ void cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                     const long long* __restrict__ targets,
                                     float* __restrict__ loss, long long rows, int vocab, int ld,
                                     float grad_scale, long long ignore_index, int* status) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __shared__ float red[33];
  const long long r = blockIdx.x;
  if (r >= rows) return;
  __nv_bfloat16* row = logits + r * (long long)ld;
  __nv_bfloat16* srow = STAGED ? reinterpret_cast<__nv_bfloat16*>(ce_smem) : row;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int nvec = ld >> 3;
  long long tgt = targets[r];
  const bool ignored = (tgt == ignore_index);
  if (!ignored && (tgt < 0 || tgt >= vocab)) {
    if (tid == 0) atomicCAS(status, 0, RT_ERR_BOUNDS);
    tgt = 0;
  }
  // Vectors [0, nfull) lie entirely inside the vocabulary, vector nfull (if vocab % 8) is cut by it, the rest is
  // padding.  Only the cut vector pays for per-element bounds tests.
  const int nfull = vocab >> 3, ncut = (vocab + 7) >> 3;
  const float LOG2E = 1.4426950408889634f;
  // pass 1: max (and stage).  Packed bf16 maxima: 4 instructions per 8 logits.
  __nv_bfloat162 m2 = __float2bfloat162_rn(-INFINITY);
  float mx = -INFINITY;
  for (int v = tid; v < ncut; v += nt) {
    uint4 w = reinterpret_cast<const uint4*>(row)[v];
    if (STAGED) reinterpret_cast<uint4*>(srow)[v] = w;
    if (v < nfull) {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
      m2 = __hmax2(m2, __hmax2(__hmax2(h2[0], h2[1]), __hmax2(h2[2], h2[3])));
    } else {
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&w);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (v * 8 + e < vocab) mx = fmaxf(mx, __bfloat162float(h[e]));
    }
  }
  mx = fmaxf(mx, fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y)));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : -INFINITY;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, s));
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  mx = red[32];
  __syncthreads();
  const float mxs = -mx * LOG2E;        // exp(x - mx) = ex2(x * log2e + mxs): one fma + one ex2 per logit
  const float xt = __bfloat162float(srow[tgt]);  // before the staged row is overwritten with its exponentials
  if (STAGED) __syncthreads();
  // pass 2: sum exp.  The staged row keeps the exponentials (bf16, the precision of the gradient that leaves anyway),
  // so the special-function unit runs once per logit instead of twice.
  float sum = 0.f;
  for (int v = tid; v < ncut; v += nt) {
    uint4 w = reinterpret_cast<const uint4*>(srow)[v];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
    if (v < nfull) {
      uint4 ex;
      uint32_t* exw = reinterpret_cast<uint32_t*>(&ex);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        const float a = ex2_approx(fmaf(f.x, LOG2E, mxs)), b = ex2_approx(fmaf(f.y, LOG2E, mxs));
        sum += a + b;
        exw[e] = pack_bf16x2(a, b);
      }
      if (STAGED) reinterpret_cast<uint4*>(srow)[v] = ex;
    } else {
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&w);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (v * 8 + e < vocab) sum += ex2_approx(fmaf(__bfloat162float(h[e]), LOG2E, mxs));
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : 0.f;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t += __shfl_xor_sync(0xffffffffu, t, s);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  sum = red[32];
  if (tid == 0) loss[r] = ignored ? 0.f : (logf(sum) + mx - xt);
  __syncthreads();  // srow[tgt] read before it is overwritten (non-staged mode aliases the row)
  const float gs = ignored ? 0.f : grad_scale;
  const float gi = gs / sum;
  // pass 3: gradient in place; the "- onehot" term is patched in afterwards by one thread
  for (int v = tid; v < nvec; v += nt) {
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (v < ncut) {
      uint4 w = reinterpret_cast<const uint4*>(srow)[v];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
      float g[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        if (STAGED && v < nfull) {      // the staged vector already holds exp(x - max)
          g[2 * e] = f.x * gi;
          g[2 * e + 1] = f.y * gi;
        } else {
          g[2 * e] = ex2_approx(fmaf(f.x, LOG2E, mxs)) * gi;
          g[2 * e + 1] = ex2_approx(fmaf(f.y, LOG2E, mxs)) * gi;
        }
      }
      if (v >= nfull) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (v * 8 + e >= vocab) g[e] = 0.f;
      }
      if (v == (int)(tgt >> 3)) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (e == (int)(tgt & 7)) g[e] -= gs;
      }
      o.x = pack_bf16x2(g[0], g[1]);
      o.y = pack_bf16x2(g[2], g[3]);
      o.z = pack_bf16x2(g[4], g[5]);
      o.w = pack_bf16x2(g[6], g[7]);
    }
    reinterpret_cast<uint4*>(row)[v] = o;
  }
}

// Register-resident variant: the whole row lives in the registers of one 1024-thread CTA as
// packed bf16 (NV 16-byte vectors per thread), so each logit is read from HBM once, exponentiated
// once (the exponentials overwrite the packed row in registers) and written once.
template <int NV>
__global__ void __launch_bounds__(1024, 1)
cross_entropy_reg_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                         float* __restrict__ loss, long long rows, int vocab, int ld,
                         float grad_scale, long long ignore_index, int* status) {
  __shared__ float red[33];
  __shared__ float s_xt;
  const long long r = blockIdx.x;
  if (r >= rows) return;
  uint4* row = reinterpret_cast<uint4*>(logits + r * (long long)ld);
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int nvec = ld >> 3;
  long long tgt = targets[r];
  const bool ignored = (tgt == ignore_index);
  if (!ignored && (tgt < 0 || tgt >= vocab)) {
    if (tid == 0) atomicCAS(status, 0, RT_ERR_BOUNDS);
    tgt = 0;
  }
  if (ignored) tgt = 0;
  uint4 w[NV];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * 1024;
    if (v < nvec) {
      w[i] = row[v];
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&w[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (v * 8 + e < vocab) mx = fmaxf(mx, __bfloat162float(h[e]));
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float t = red[lane];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, s));
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  mx = red[32];
  __syncthreads();
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * 1024;
    if (v < nvec) {
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&w[i]);
      float ev[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int c = v * 8 + e;
        const float x = __bfloat162float(h[e]);
        if (c == tgt) s_xt = x;
        ev[e] = (c < vocab) ? __expf(x - mx) : 0.f;
        sum += ev[e];
      }
      w[i].x = pack_bf16x2(ev[0], ev[1]);
      w[i].y = pack_bf16x2(ev[2], ev[3]);
      w[i].z = pack_bf16x2(ev[4], ev[5]);
      w[i].w = pack_bf16x2(ev[6], ev[7]);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float t = red[lane];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t += __shfl_xor_sync(0xffffffffu, t, s);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  sum = red[32];
  const float inv = 1.f / sum;
  if (tid == 0) loss[r] = ignored ? 0.f : (logf(sum) + mx - s_xt);
  const float gs = ignored ? 0.f : grad_scale;
  const float gi = inv * gs;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * 1024;
    if (v < nvec) {
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&w[i]);
      float g[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int c = v * 8 + e;
        g[e] = __bfloat162float(h[e]) * gi - ((c == tgt) ? gs : 0.f);
      }
      uint4 o;
      o.x = pack_bf16x2(g[0], g[1]);
      o.y = pack_bf16x2(g[2], g[3]);
      o.z = pack_bf16x2(g[4], g[5]);
      o.w = pack_bf16x2(g[6], g[7]);
      row[v] = o;
    }
  }
}

void cross_entropy_fwd_bwd(void* logits, const long long* targets, float* loss, long long rows,
                           int vocab, int ld, float grad_scale, long long ignore_index,
                           cudaStream_t stream) {
  RT_CHECK(ld % 8 == 0 && ld >= vocab, "cross_entropy: row stride must be a multiple of 8 and >= vocab");
  if (rows == 0) return;
  const int device = current_device();
  const size_t need = (size_t)ld * 2;
  auto lg = reinterpret_cast<__nv_bfloat16*>(logits);
  const int nvec = ld >> 3;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (need <= 110 * 1024) {
    static bool configured[64] = {false};
    if (!configured[device]) {
      RT_CUDA_CHECK(cudaFuncSetAttribute(cross_entropy_kernel<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
      configured[device] = true;
    }
    cross_entropy_kernel<true><<<(unsigned)rows, 512, need, stream>>>(
        lg, targets, loss, rows, vocab, ld, grad_scale, ignore_index, status_word(device));
  } else if (aligned && nvec <= 8 * 1024) {
    cross_entropy_reg_kernel<8><<<(unsigned)rows, 1024, 0, stream>>>(
        lg, targets, loss, rows, vocab, ld, grad_scale, ignore_index, status_word(device));
  } else if (aligned && nvec <= 16 * 1024) {
    cross_entropy_reg_kernel<16><<<(unsigned)rows, 1024, 0, stream>>>(
        lg, targets, loss, rows, vocab, ld, grad_scale, ignore_index, status_word(device));
  } else {
    cross_entropy_kernel<false><<<(unsigned)rows, 512, 0, stream>>>(
        lg, targets, loss, rows, vocab, ld, grad_scale, ignore_index, status_word(device));
  }
  RT_LAUNCH_CHECK();
}

}  // namespace rt
