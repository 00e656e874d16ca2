// fp16 inference kernels of the LLM runtime (Llama-family decode / prefill with a KV cache):
//   rmsnorm_f16          y = x * rsqrt(mean(x^2) + eps) * w
//   rope_kv_f16          rotary embedding on q and k in place (adjacent pairs (2i, 2i+1) as GGUF llama
//                        weights expect, or half-split pairs (i, i + D/2)) and append of the new k / v rows
//                        to the cache
//   attn_cache_f16       softmax(q K^T / sqrt(D)) V over the cached keys, one CTA per (query, head);
//                        query i attends to cache positions [0, kv_len[i])  (causal by construction)
//   silu_mul_f16         SwiGLU gate: silu(gate) * up
// The reference's runtime re-runs the whole sequence per generated token with scalar host loops and no
// KV cache (example-cli/src/model/inference.rs:135-192, model/architectures/attention.rs:233-303); its
// KVCache struct is unused (model/transformer.rs:221-270).
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

__global__ void rmsnorm_f16_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                   __half* __restrict__ y, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  const __half2* xr = reinterpret_cast<const __half2*>(x + row * C);
  __shared__ float red[32];
  float ss = 0.f;
  for (int i = threadIdx.x; i < (C >> 1); i += blockDim.x) {
    const float2 f = __half22float2(xr[i]);
    ss += f.x * f.x + f.y * f.y;
  }
  ss = wsum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = wsum(t);
    if (threadIdx.x == 0) red[0] = rsqrtf(t / C + eps);
  }
  __syncthreads();
  const float r = red[0];
  const __half2* wr = reinterpret_cast<const __half2*>(w);
  __half2* yr = reinterpret_cast<__half2*>(y + row * C);
  for (int i = threadIdx.x; i < (C >> 1); i += blockDim.x) {
    const float2 f = __half22float2(xr[i]), g = __half22float2(wr[i]);
    yr[i] = __floats2half2_rn(f.x * r * g.x, f.y * r * g.y);
  }
}

// q: [n_tok][H][D], k/v: [n_tok][Hkv][D] (rows of the fused qkv output, strides in halves).
// cache_k / cache_v: [B][Hkv][T_max][D].  Token t belongs to sequence seq[t] at position pos[t].
// grid (n_tok, H + 2 Hkv): blockIdx.y selects a q head, a k head (rotated and appended to the cache) or a
// v head (appended).  One thread per rotation pair; a token with one CTA per head keeps the step short
// for decode, where n_tok is the batch size.
__global__ void rope_kv_f16_kernel(__half* __restrict__ q, long long q_st, __half* __restrict__ k,
                                   long long k_st, const __half* __restrict__ v, long long v_st,
                                   __half* __restrict__ cache_k, __half* __restrict__ cache_v,
                                   const int* __restrict__ pos, const int* __restrict__ seq, int H, int Hkv,
                                   int D, int T_max, float log2_theta, int interleaved, int n_seq, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, hy = blockIdx.y;
  const int p = pos[t], s = seq[t];
  // position and sequence number come from device data (a replayed decode graph advances them itself): a step past
  // the end of the cache is reported, not written
  if (p < 0 || p >= T_max || s < 0 || s >= n_seq) {
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BOUNDS);
    return;
  }
  const int half_d = D >> 1;
  if (hy >= H + Hkv) {  // v head: plain append
    const int h = hy - H - Hkv;
    const __half2* src = reinterpret_cast<const __half2*>(v + t * v_st + h * D);
    __half2* dst = reinterpret_cast<__half2*>(cache_v + (((long long)s * Hkv + h) * T_max + p) * D);
    for (int d = threadIdx.x; d < half_d; d += blockDim.x) dst[d] = src[d];
    return;
  }
  const bool is_q = hy < H;
  const int h = is_q ? hy : hy - H;
  __half* base = is_q ? q + t * q_st + h * D : k + t * k_st + h * D;
  __half* ck = is_q ? nullptr : cache_k + (((long long)s * Hkv + h) * T_max + p) * D;
  for (int d = threadIdx.x; d < half_d; d += blockDim.x) {
    const float inv_freq = exp2f(-2.f * (float)d / (float)D * log2_theta);
    float sn, cs;
    sincosf((float)p * inv_freq, &sn, &cs);
    const int ia = interleaved ? 2 * d : d, ib = interleaved ? 2 * d + 1 : d + half_d;
    const float a = __half2float(base[ia]), b = __half2float(base[ib]);
    const __half ra = __float2half(a * cs - b * sn), rb = __float2half(a * sn + b * cs);
    base[ia] = ra;
    base[ib] = rb;
    if (ck) {
      ck[ia] = ra;
      ck[ib] = rb;
    }
  }
}

// One CTA (128 threads) per (query token, head).  Scores live in shared memory (kv_len floats).
__global__ void attn_cache_f16_kernel(const __half* __restrict__ q, long long q_st,
                                      const __half* __restrict__ cache_k, const __half* __restrict__ cache_v,
                                      __half* __restrict__ out, long long o_st, const int* __restrict__ kv_len,
                                      const int* __restrict__ seq, int H, int Hkv, int D, int T_max, float scale) {
  extern __shared__ float sc[];  // [kv_len] scores, then [4][D] partial outputs
  __shared__ float red[8];
  const int t = blockIdx.x, h = blockIdx.y;
  const int hk = h / (H / Hkv);
  const int L = kv_len[t], s = seq[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const __half* qv = q + t * q_st + h * D;
  const __half* K = cache_k + ((long long)s * Hkv + hk) * T_max * D;
  const __half* V = cache_v + ((long long)s * Hkv + hk) * T_max * D;
  // each lane keeps its slice of q (D <= 256: up to 8 halves per lane)
  float qr[8];
  const int per_lane = D / 32;
#pragma unroll
  for (int e = 0; e < 8; ++e) qr[e] = e < per_lane ? __half2float(qv[lane * per_lane + e]) * scale : 0.f;
  float mx = -INFINITY;
  for (int j = warp; j < L; j += nw) {
    const __half* kr = K + (long long)j * D + lane * per_lane;
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (e < per_lane) dot += qr[e] * __half2float(kr[e]);
    dot = wsum(dot);
    if (lane == 0) sc[j] = dot;
    mx = fmaxf(mx, dot);
  }
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < nw; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < L; j += blockDim.x) {
    const float e = __expf(sc[j] - mx);
    sc[j] = e;
    sum += e;
  }
  sum = wsum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < nw; ++w) sum += red[w];
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  // O = P V : thread d accumulates output dim d over a strided subset of keys, partials merged in smem
  float* part = sc + ((L + 3) & ~3);
  const int groups = blockDim.x / D > 0 ? blockDim.x / D : 1;  // key groups working in parallel
  const int d = threadIdx.x % D, g = threadIdx.x / D;
  if (threadIdx.x < groups * D) {
    float acc = 0.f;
    for (int j = g; j < L; j += groups) acc += sc[j] * __half2float(V[(long long)j * D + d]);
    part[g * D + d] = acc;
  }
  __syncthreads();
  if (threadIdx.x < D) {
    float acc = 0.f;
    for (int gg = 0; gg < groups; ++gg) acc += part[gg * D + threadIdx.x];
    out[t * o_st + h * D + threadIdx.x] = __float2half(acc * inv);
  }
}

__global__ void silu_mul_f16_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                    __half* __restrict__ out, long long n2, long long g_ld, long long u_ld,
                                    long long o_ld, int cols2) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const long long r = i / cols2, c = i % cols2;
  const float2 g = __half22float2(reinterpret_cast<const __half2*>(gate + r * g_ld)[c]);
  const float2 u = __half22float2(reinterpret_cast<const __half2*>(up + r * u_ld)[c]);
  reinterpret_cast<__half2*>(out + r * o_ld)[c] =
      __floats2half2_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
}

void rmsnorm_f16(const void* x, const void* w, void* y, long long rows, int C, float eps, cudaStream_t s) {
  RT_CHECK(C % 2 == 0, "rmsnorm_f16: feature size must be even");
  if (rows == 0) return;
  launch_pdl(rmsnorm_f16_kernel, dim3((unsigned)rows), dim3(256), 0, s, reinterpret_cast<const __half*>(x),
             reinterpret_cast<const __half*>(w), reinterpret_cast<__half*>(y), C, eps);
  RT_LAUNCH_CHECK();
}

void rope_kv_f16(const RopeKvArgs& a, cudaStream_t s) {
  RT_CHECK(a.D % 2 == 0, "rope: head_dim must be even");
  RT_CHECK(a.n_seq >= 1, "rope: the cache holds no sequence");
  if (a.n_tok == 0) return;
  const int threads = std::min(128, std::max(32, ((a.D / 2 + 31) / 32) * 32));
  launch_pdl(rope_kv_f16_kernel, dim3(a.n_tok, a.H + 2 * a.Hkv), dim3(threads), 0, s, reinterpret_cast<__half*>(a.q), a.q_st,
             reinterpret_cast<__half*>(a.k), a.k_st, reinterpret_cast<const __half*>(a.v), a.v_st,
             reinterpret_cast<__half*>(a.cache_k), reinterpret_cast<__half*>(a.cache_v), a.pos, a.seq, a.H, a.Hkv, a.D, a.T_max,
             log2f(a.theta), a.interleaved, a.n_seq, status_word(current_device()));
  RT_LAUNCH_CHECK();
}

void attn_cache_f16(const AttnCacheArgs& a, cudaStream_t s) {
  RT_CHECK(a.D % 32 == 0 && a.D <= 256, "attn_cache: head_dim must be a multiple of 32 and <= 256");
  if (a.n_tok == 0) return;
  const int threads = a.D <= 128 ? 128 : 256;
  const int groups = threads / a.D > 0 ? threads / a.D : 1;
  const size_t smem = sizeof(float) * (((size_t)a.max_kv_len + 3) / 4 * 4 + (size_t)groups * a.D);
  RT_CHECK(smem <= 200 * 1024, "attn_cache: kv length too large for the shared-memory score buffer");
  if (smem > 48 * 1024)
    RT_CUDA_CHECK(cudaFuncSetAttribute(attn_cache_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.n_tok, a.H);
  attn_cache_f16_kernel<<<grid, threads, smem, s>>>(
      reinterpret_cast<const __half*>(a.q), a.q_st, reinterpret_cast<const __half*>(a.cache_k),
      reinterpret_cast<const __half*>(a.cache_v), reinterpret_cast<__half*>(a.out), a.o_st, a.kv_len, a.seq, a.H,
      a.Hkv, a.D, a.T_max, a.scale);
  RT_LAUNCH_CHECK();
}

void silu_mul_f16(const void* gate, const void* up, void* out, long long rows, int cols, long long g_ld,
                  long long u_ld, long long o_ld, cudaStream_t s) {
  RT_CHECK(cols % 2 == 0 && g_ld % 2 == 0 && u_ld % 2 == 0 && o_ld % 2 == 0, "silu_mul: even sizes required");
  const long long n2 = rows * (cols / 2);
  if (n2 == 0) return;
  launch_pdl(silu_mul_f16_kernel, dim3((unsigned)((n2 + 255) / 256)), dim3(256), 0, s, reinterpret_cast<const __half*>(gate),
             reinterpret_cast<const __half*>(up), reinterpret_cast<__half*>(out), n2, g_ld, u_ld, o_ld, cols / 2);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
