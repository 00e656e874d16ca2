// Data-parallel gradient bucket step in ONE kernel over NVLink peer memory:
//
//   start barrier (flags in peer memory)                         "bucket gradients are final on every rank"
//   for the 1/N shard of the bucket this rank owns:
//     g  = (1/N) * sum over ranks of grad_rank[i]                 P2P loads (plain ld, L2-only)
//     peers' and own grad[i] = 0                                 P2P stores (ready for the next backward)
//     AdamW(master, m, v, g)                                     fp32, local
//     every rank's bf16 parameter copy[i] = bf16(master[i])      P2P stores (the all-gather half)
//   end signal (flags in peer memory)                            "my writes into your buffers are done"
//
// i.e. reduce-scatter + scale + optimizer + all-gather with no intermediate buffer and no separate
// collective launch.  It replaces the reference's per-parameter all_reduce loop, whose
// collective is a no-op stub (src/distributed/ddp.rs:156-172, src/distributed/common.rs:49-56),
// and its 25 MB bucket plan (src/distributed/ddp.rs:235-271).
//
// Peer access is by plain loads/stores on peer pointers from symmetric allocations; there is no
// TMA and no multicast in this file.  Each thread keeps 8 sixteen-byte loads in flight, so a 25 MB
// bucket streams at memory / link speed for a few tens of microseconds and the backward kernels
// it overlaps lose little.
// Every wait is bounded by a caller-supplied deadline; on expiry the kernel records
// RT_ERR_TIMEOUT_PEER in the status word, skips its update and returns.
#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Wait until flags[i] >= epoch for every i in [0, n) except `skip`.  Returns false on timeout.
__device__ __forceinline__ bool wait_flags(const int* flags, int n, int skip, int epoch,
                                           unsigned long long timeout_ns, int* status) {
  bool ok = true;
  if (threadIdx.x < n && int(threadIdx.x) != skip) {
    const int* f = flags + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    unsigned it = 0;
    while (ld_acquire_sys(f) < epoch) {
      if ((++it & 0x3ff) == 0 && globaltimer_ns() - t0 > timeout_ns) {
        atomicCAS(status, 0, RT_ERR_TIMEOUT_PEER);
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__device__ __forceinline__ void adamw4(const DdpBucketArgs& a, float4& pm, const float4& g, float4& m,
                                       float4& v) {
  const float inv_w = a.grad_scale;
#define RT_ADAMW1(P, G, M, V)                                          \
  {                                                                    \
    const float gg = (G) * inv_w;                                      \
    (M) = a.beta1 * (M) + (1.f - a.beta1) * gg;                        \
    (V) = a.beta2 * (V) + (1.f - a.beta2) * gg * gg;                   \
    (P) *= (1.f - a.lr * a.weight_decay);                              \
    (P) -= a.lr * ((M) / a.bias_corr1) / (sqrtf((V) / a.bias_corr2) + a.eps); \
  }
  RT_ADAMW1(pm.x, g.x, m.x, v.x)
  RT_ADAMW1(pm.y, g.y, m.y, v.y)
  RT_ADAMW1(pm.z, g.z, m.z, v.z)
  RT_ADAMW1(pm.w, g.w, m.w, v.w)
#undef RT_ADAMW1
}

// WT = compile-time world size (1, 2, 4, 8) or 0 for "read it from the arguments".  Each thread
// handles G = 8 / WT groups of 4 elements per trip and issues the G x W peer loads before it
// consumes any, i.e. 8 sixteen-byte loads in flight per thread whatever the world size.
template <int WT>
__global__ void __launch_bounds__(256, 2) ddp_bucket_adamw_kernel(const DdpBucketArgs a) {
  const int W = WT > 0 ? WT : a.world;
  const int R = a.rank;
  constexpr int G = WT > 0 ? 8 / WT : 1;
  constexpr int WMAX = WT > 0 ? WT : RT_MAX_PEERS;
  int* my_flags = a.flags[R];
  // ---- start barrier: tell every peer this rank's bucket gradients are final, wait for theirs
  if (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x < W && int(threadIdx.x) != R) {
      __threadfence_system();
      st_release_sys(a.flags[threadIdx.x] + a.start_slot + R, a.epoch);
    }
    if (!wait_flags(my_flags + a.start_slot, W, R, a.epoch, a.timeout_ns, a.status)) return;
  }

  const long long base = a.bucket_start + (long long)R * a.chunk_len;  // flat index of my shard
  const long long n4 = a.chunk_len >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += G * stride) {
    float4 v[G][WMAX];
    long long e[G];
    bool on[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long i = i0 + g * stride;
      on[g] = i < n4;
      e[g] = base + ((on[g] ? i : i0) << 2);
#pragma unroll
      for (int p = 0; p < WMAX; ++p)
        if (p < W && on[g]) v[g][p] = ld_peer_f4(a.grad[p] + e[g]);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!on[g]) continue;
      float4 sum = z;
#pragma unroll
      for (int p = 0; p < WMAX; ++p) {
        if (p < W) {
          sum.x += v[g][p].x; sum.y += v[g][p].y; sum.z += v[g][p].z; sum.w += v[g][p].w;
          *reinterpret_cast<float4*>(a.grad[p] + e[g]) = z;
        }
      }
      float4 pm = *reinterpret_cast<float4*>(a.master + e[g]);
      float4 m = *reinterpret_cast<float4*>(a.m + e[g]);
      float4 vv = *reinterpret_cast<float4*>(a.v + e[g]);
      adamw4(a, pm, sum, m, vv);
      *reinterpret_cast<float4*>(a.master + e[g]) = pm;
      *reinterpret_cast<float4*>(a.m + e[g]) = m;
      *reinterpret_cast<float4*>(a.v + e[g]) = vv;
      uint2 w;
      w.x = pack_bf16x2(pm.x, pm.y);
      w.y = pack_bf16x2(pm.z, pm.w);
#pragma unroll
      for (int p = 0; p < WMAX; ++p)
        if (p < W) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.lp[p]) + e[g]) = w;
    }
  }

  // ---- end signal: the last CTA to finish tells every peer that this rank is done writing
  if (W > 1) {
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(a.done_counter, 1u);
      s_last = (prev == gridDim.x - 1) ? 1 : 0;
      if (s_last) *a.done_counter = 0;  // re-armed for the next launch that uses this counter
    }
    __syncthreads();
    if (s_last && threadIdx.x < W && int(threadIdx.x) != R) {
      __threadfence_system();
      st_release_sys(a.flags[threadIdx.x] + a.end_slot + R, a.epoch);
    }
  }
}

// Waits until every peer has signalled the end of every bucket of this step.
__global__ void ddp_wait_end_kernel(const int* flags, int n_slots, int world, int rank, int epoch,
                                    unsigned long long timeout_ns, int* status) {
  // flags layout: slot s, source rank p  ->  flags[s * world + p]
  for (int s = 0; s < n_slots; ++s) {
    if (!wait_flags(flags + (long long)s * world, world, rank, epoch, timeout_ns, status)) return;
  }
}

void ddp_bucket_adamw(const DdpBucketArgs& a, int n_ctas, cudaStream_t stream) {
  RT_CHECK(a.world >= 1 && a.world <= RT_MAX_PEERS, "ddp: world size must be in [1, 8]");
  RT_CHECK(a.chunk_len % 4 == 0 && a.bucket_start % 4 == 0, "ddp: bucket geometry must be 4-aligned");
  if (a.chunk_len == 0) return;
  switch (a.world) {
    case 1: ddp_bucket_adamw_kernel<1><<<n_ctas, 256, 0, stream>>>(a); break;
    case 2: ddp_bucket_adamw_kernel<2><<<n_ctas, 256, 0, stream>>>(a); break;
    case 4: ddp_bucket_adamw_kernel<4><<<n_ctas, 256, 0, stream>>>(a); break;
    case 8: ddp_bucket_adamw_kernel<8><<<n_ctas, 256, 0, stream>>>(a); break;
    default: ddp_bucket_adamw_kernel<0><<<n_ctas, 256, 0, stream>>>(a); break;
  }
  RT_LAUNCH_CHECK();
}

void ddp_wait_end(const int* flags, int n_slots, int world, int rank, int epoch,
                  unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  if (world <= 1 || n_slots == 0) return;
  ddp_wait_end_kernel<<<1, 32, 0, stream>>>(flags, n_slots, world, rank, epoch, timeout_ns, status);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
