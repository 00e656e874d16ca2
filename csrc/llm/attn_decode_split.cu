// Split-KV attention over a KV cache for decode and short prefill (fp16, online softmax):
//
//   out[t][h] = softmax(q[t][h] . K[seq[t]][h / G][0 .. kv_len[t]) * scale) V[...]
//
// A decode step has only batch x heads independent rows, far fewer than 148 SMs can hide HBM latency
// with, so the key range of every (token, kv head) is cut into `n_split` slices handled by separate CTAs
// (grid = tokens x kv heads x slices); the slices' (max, sum, acc) triples meet in a global scratch and the CTA
// that arrives last at a per-(token, kv head) counter merges them and re-arms the counter, so the step is one
// launch.  Inside a CTA a key row of D halves is read by D/8 lanes with one 16-byte load each, so a warp
// covers 32/(D/8) keys per step and keeps UN steps of K and V loads in flight; all G = H/Hkv query heads
// that share the kv head are served from the same K/V registers (grouped-query attention reads the cache
// once).  Each (warp, key slot) keeps its own running softmax state, merged once at the end: no
// shuffles or barriers on the critical path of the key loop apart from the D/8-lane dot-product reduce.
//
// The reference has no KV-cache attention at all (its KVCache type is unused,
// example-cli/src/model/transformer.rs:221-270; attention is a scalar host loop over the whole
// sequence per generated token, model/architectures/attention.rs:233-303).
#include <cuda_fp16.h>
#include <math_constants.h>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

constexpr int ADS_WARPS = 4;
constexpr int ADS_UN = 8;

__device__ __forceinline__ uint4 ld16(const __half* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// Merge softmax state (mo, lo, ao) into (m, l, a); states with m = -inf are empty.
__device__ __forceinline__ void merge_state(float& m, float& l, float (&a)[8], float mo, float lo, const float (&ao)[8]) {
  const float mn = fmaxf(m, mo);
  if (mn == -CUDART_INF_F) return;
  const float ca = exp2f(m - mn), cb = exp2f(mo - mn);
  l = l * ca + lo * cb;
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = a[e] * ca + ao[e] * cb;
  m = mn;
}

template <int D, int G>
__global__ void __launch_bounds__(ADS_WARPS * 32)
attn_decode_split_kernel(const __half* __restrict__ q, long long q_st, const __half* __restrict__ cache_k,
                         const __half* __restrict__ cache_v, __half* __restrict__ out, long long o_st,
                         const int* __restrict__ kv_len, const int* __restrict__ seq, int H, int Hkv, int T_max,
                         float scale_log2, int n_split, float* __restrict__ part, int* __restrict__ counters, int n_seq,
                         int* __restrict__ status) {
  constexpr int LPK = D / 8;    // lanes per key row
  constexpr int KPW = 32 / LPK; // keys per warp step
  __shared__ float sm_acc[ADS_WARPS][G][D];
  __shared__ float sm_ml[ADS_WARPS][G][2];
  __shared__ int sm_last;
  pdl_launch_dependents();
  pdl_wait();

  const int t = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  int L = kv_len[t];
  const int s = seq[t];
  // both come from device data: a length past the cache or a foreign sequence number is reported and made harmless
  if (L > T_max || L < 0 || s < 0 || s >= n_seq) {
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BOUNDS);
    L = (s < 0 || s >= n_seq) ? 0 : min(max(L, 0), T_max);
  }
  const int s_safe = (s < 0 || s >= n_seq) ? 0 : s;
  const int per = (L + n_split - 1) / n_split;
  const int j0 = sp * per, j1 = min(L, j0 + per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, dl = lane % LPK;
  const __half* K = cache_k + ((long long)s_safe * Hkv + hk) * T_max * D + dl * 8;
  const __half* V = cache_v + ((long long)s_safe * Hkv + hk) * T_max * D + dl * 8;

  float qr[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    unpack8(ld16(q + t * q_st + (long long)(hk * G + g) * D + dl * 8), qr[g]);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      qr[g][e] *= scale_log2;
      acc[g][e] = 0.f;
    }
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
  }

  for (int base = j0 + warp * KPW; base < j1; base += ADS_WARPS * KPW * ADS_UN) {
    uint4 kraw[ADS_UN], vraw[ADS_UN];
#pragma unroll
    for (int u = 0; u < ADS_UN; ++u) {
      const int j = base + u * ADS_WARPS * KPW + sub;
      if (j < j1) {
        kraw[u] = ld16(K + (long long)j * D);
        vraw[u] = ld16(V + (long long)j * D);
      } else {
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < ADS_UN; ++u) {
      const int j = base + u * ADS_WARPS * KPW + sub;
      float kf[8], vf[8];
      unpack8(kraw[u], kf);
      unpack8(vraw[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qr[g][e], kf[e], dot);
#pragma unroll
        for (int o = LPK >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (j < j1) {
          const float mn = fmaxf(m[g], dot);
          const float corr = exp2f(m[g] - mn), p = exp2f(dot - mn);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(acc[g][e], corr, p * vf[e]);
          m[g] = mn;
        }
      }
    }
  }

  // merge the key slots of the warp, then the warps of the CTA
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      float ao[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) ao[e] = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
      merge_state(m[g], l[g], acc[g], mo, lo, ao);
    }
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sm_acc[warp][g][dl * 8 + e] = acc[g][e];
      if (dl == 0) {
        sm_ml[warp][g][0] = m[g];
        sm_ml[warp][g][1] = l[g];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < ADS_WARPS; ++w) mm = fmaxf(mm, sm_ml[w][g][0]);
    float a = 0.f, ll = 0.f;
    if (mm != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < ADS_WARPS; ++w) {
        const float c = exp2f(sm_ml[w][g][0] - mm);
        a += sm_acc[w][g][d] * c;
        ll += sm_ml[w][g][1] * c;
      }
    }
    const int h = hk * G + g;
    if (n_split == 1) {
      out[t * o_st + (long long)h * D + d] = __float2half(ll > 0.f ? a / ll : 0.f);
    } else {
      float* dst = part + (((long long)t * H + h) * n_split + sp) * (D + 2);
      dst[d] = a;
      if (d == 0) {
        dst[D] = mm;
        dst[D + 1] = ll;
      }
    }
  }
  if (n_split == 1) return;
  // last slice to arrive merges all slices of this (token, kv head)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&counters[t * Hkv + hk], 1);
    sm_last = (prev == n_split - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    const int h = hk * G + g;
    const float* src = part + ((long long)t * H + h) * n_split * (D + 2);
    float mm = -CUDART_INF_F;
    for (int k = 0; k < n_split; ++k) mm = fmaxf(mm, __ldcg(src + k * (D + 2) + D));
    float a = 0.f, ll = 0.f;
    if (mm != -CUDART_INF_F) {
      for (int k = 0; k < n_split; ++k) {
        const float c = exp2f(__ldcg(src + k * (D + 2) + D) - mm);
        a += __ldcg(src + k * (D + 2) + d) * c;
        ll += __ldcg(src + k * (D + 2) + D + 1) * c;
      }
    }
    out[t * o_st + (long long)h * D + d] = __float2half(ll > 0.f ? a / ll : 0.f);
  }
  if (threadIdx.x == 0) counters[t * Hkv + hk] = 0;  // re-armed for the next call on this stream
}

template <int D, int G>
void launch_split(const AttnCacheArgs& a, cudaStream_t s) {
  dim3 grid(a.n_tok, a.Hkv, a.n_split);
  launch_pdl(attn_decode_split_kernel<D, G>, grid, dim3(ADS_WARPS * 32), 0, s, reinterpret_cast<const __half*>(a.q), a.q_st,
             reinterpret_cast<const __half*>(a.cache_k), reinterpret_cast<const __half*>(a.cache_v), reinterpret_cast<__half*>(a.out),
             a.o_st, a.kv_len, a.seq, a.H, a.Hkv, a.T_max, a.scale * 1.4426950408889634f, a.n_split, a.partial, a.counters, a.n_seq,
             status_word(current_device()));
  RT_LAUNCH_CHECK();
}

template <int D>
bool dispatch_g(const AttnCacheArgs& a, cudaStream_t s) {
  switch (a.H / a.Hkv) {
    case 1: launch_split<D, 1>(a, s); return true;
    case 2: launch_split<D, 2>(a, s); return true;
    case 4: launch_split<D, 4>(a, s); return true;
    case 8: launch_split<D, 8>(a, s); return true;
    default: return false;
  }
}

}  // namespace

bool attn_decode_split_supported(int D, int H, int Hkv) {
  const int g = Hkv > 0 && H % Hkv == 0 ? H / Hkv : 0;
  return (D == 64 || D == 128 || D == 256) && (g == 1 || g == 2 || g == 4 || g == 8);
}

// Number of key slices: enough CTAs for four per SM (a slice is then a handful of loads deep: the kernel is bound
// by dependent-load latency, not bandwidth), but at least 32 keys per slice.
int attn_decode_num_splits(int n_tok, int Hkv, int max_kv_len, int sm_count) {
  const long long rows = (long long)n_tok * Hkv;
  long long want = (4LL * sm_count + rows - 1) / rows;
  const long long cap = (max_kv_len + 31) / 32;
  if (want > cap) want = cap;
  if (want > 64) want = 64;
  return want < 1 ? 1 : (int)want;
}

void attn_decode_split(const AttnCacheArgs& a, cudaStream_t s) {
  RT_CHECK(attn_decode_split_supported(a.D, a.H, a.Hkv), "attn_decode_split: unsupported head_dim / group size");
  RT_CHECK(a.n_split >= 1 && (a.n_split == 1 || (a.partial != nullptr && a.counters != nullptr)),
           "attn_decode_split: partial buffer and zeroed counters required");
  RT_CHECK(a.q_st % 8 == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0, "attn_decode_split: q must be 16-byte aligned");
  if (a.n_tok == 0) return;
  bool ok = false;
  if (a.D == 64) ok = dispatch_g<64>(a, s);
  else if (a.D == 128) ok = dispatch_g<128>(a, s);
  else ok = dispatch_g<256>(a, s);
  RT_CHECK(ok, "attn_decode_split: dispatch failed");
}

}  // namespace rt
