// Token + learned-position embedding lookup (forward) and its scatter-add backward.
// The reference's Embedding / PositionalEmbedding are forward-only host loops
// (src/nn/embedding.rs:18-607); GPT sums the two lookups (src/models/transformer_models.rs:760-796).
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

// out[r][:] = wte[idx[r]][:] (+ wpe[r % T][:])   one block per row, 16-byte vectors.
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx,
                                     const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe,
                                     __nv_bfloat16* __restrict__ out, long long rows, int T, int C,
                                     int vocab, int* status) {
  const long long r = blockIdx.x;
  if (r >= rows) return;
  long long tok = idx[r];
  if (tok < 0 || tok >= vocab) {  // record and clamp instead of faulting
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BOUNDS);
    tok = tok < 0 ? 0 : vocab - 1;
  }
  const uint4* te = reinterpret_cast<const uint4*>(wte + tok * C);
  const uint4* pe = wpe ? reinterpret_cast<const uint4*>(wpe + (r % T) * C) : nullptr;
  uint4* o = reinterpret_cast<uint4*>(out + r * C);
  for (int v = threadIdx.x; v < (C >> 3); v += blockDim.x) {
    uint4 a = te[v];
    if (pe) {
      uint4 b = pe[v];
      __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 x = __bfloat1622float2(ha[e]), y = __bfloat1622float2(hb[e]);
        ha[e] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
      }
    }
    o[v] = a;
  }
}

// dwte[idx[r]][:] += dout[r][:] ; dwpe[r % T][:] += dout[r][:]   (fp32 atomics)
__global__ void embedding_bwd_kernel(const long long* __restrict__ idx,
                                     const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dwte, float* __restrict__ dwpe,
                                     long long rows, int T, int C, int vocab) {
  const long long r = blockIdx.x;
  if (r >= rows) return;
  long long tok = idx[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __nv_bfloat162* d = reinterpret_cast<const __nv_bfloat162*>(dout + r * C);
  float* te = dwte ? dwte + tok * C : nullptr;
  float* pe = dwpe ? dwpe + (r % T) * C : nullptr;
  for (int v = threadIdx.x; v < (C >> 1); v += blockDim.x) {
    float2 g = __bfloat1622float2(d[v]);
    if (te) {
      atomicAdd(te + 2 * v, g.x);
      atomicAdd(te + 2 * v + 1, g.y);
    }
    if (pe) {
      atomicAdd(pe + 2 * v, g.x);
      atomicAdd(pe + 2 * v + 1, g.y);
    }
  }
}

void embedding_fwd(const long long* idx, const void* wte, const void* wpe, void* out,
                   long long rows, int T, int C, int vocab, cudaStream_t stream) {
  RT_CHECK(C % 8 == 0, "embedding: dim must be a multiple of 8");
  if (rows == 0) return;
  embedding_fwd_kernel<<<(unsigned)rows, 128, 0, stream>>>(
      idx, reinterpret_cast<const __nv_bfloat16*>(wte), reinterpret_cast<const __nv_bfloat16*>(wpe),
      reinterpret_cast<__nv_bfloat16*>(out), rows, T, C, vocab, status_word(current_device()));
  RT_LAUNCH_CHECK();
}

void embedding_bwd(const long long* idx, const void* dout, float* dwte, float* dwpe,
                   long long rows, int T, int C, int vocab, cudaStream_t stream) {
  if (rows == 0) return;
  embedding_bwd_kernel<<<(unsigned)rows, 128, 0, stream>>>(
      idx, reinterpret_cast<const __nv_bfloat16*>(dout), dwte, dwpe, rows, T, C, vocab);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
