// Data-parallel gradient bucket step in ONE kernel over NVLink peer memory:
//
//   start barrier (flags in peer memory)                         "bucket gradients are final on every rank"
//   for the 1/N shard of the bucket this rank owns:
//     g  = (1/N) * sum over ranks of grad_rank[i]                 P2P loads, or ONE multimem.ld_reduce (NVLS)
//     own grad[i] = 0                                            local (each rank zeroes the rest of its buffer itself after the step)
//     AdamW / Adam / SGD-momentum(master, m, v, g)               fp32, local
//     every rank's bf16 parameter copy[i] = bf16(master[i])      P2P stores, or one multimem.st
//   end signal (flags in peer memory)                            "my writes into your buffers are done"
//
// i.e. reduce-scatter + scale + optimizer + all-gather with no intermediate buffer and no separate
// collective launch.  It replaces the reference's per-parameter all_reduce loop, whose
// collective is a no-op stub (src/distributed/ddp.rs:156-172, src/distributed/common.rs:49-56),
// and its 25 MB bucket plan (src/distributed/ddp.rs:235-271).
//
// Peer access is by plain loads/stores on peer pointers from symmetric allocations or, when the caller
// passes the multicast mapping of the same allocations, by multimem instructions that the NVSwitch
// reduces / replicates (each element then crosses this GPU's links once per direction instead of N - 1
// times); there is no TMA in this file.  Each thread keeps 8 sixteen-byte loads in flight, so a 25 MB
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

// Multicast (NVLS) accessors: one instruction acts on the same offset of EVERY rank's buffer through the
// NVSwitch.  ld_reduce returns the sum over all ranks (the switch adds), st writes all ranks' copies.
__device__ __forceinline__ float4 mc_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_b32x2(void* mc, uint32_t lo, uint32_t hi) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "f"(__uint_as_float(lo)),
               "f"(__uint_as_float(hi))
               : "memory");
}

// One element of the update rule selected by a.opt_mode (same arithmetic as optim/fused_optim.cu).
__device__ __forceinline__ void ddp_update1(const DdpBucketArgs& a, float& p, float g, float& m, float& v) {
  g *= a.grad_scale;
  if (a.opt_mode == OPT_SGD) {  // beta1 = momentum, beta2 = dampening, L2 decay in the gradient
    g += a.weight_decay * p;
    float d = g;
    if (a.beta1 != 0.f) {
      m = a.first_step ? g : (a.beta1 * m + (1.f - a.beta2) * g);
      d = a.nesterov ? (g + a.beta1 * m) : m;
    }
    p -= a.lr * d;
  } else {
    if (a.opt_mode == OPT_ADAM) g += a.weight_decay * p;
    m = a.beta1 * m + (1.f - a.beta1) * g;
    v = a.beta2 * v + (1.f - a.beta2) * g * g;
    if (a.opt_mode == OPT_ADAMW) p *= (1.f - a.lr * a.weight_decay);
    p -= a.lr * (m / a.bias_corr1) / (sqrtf(v / a.bias_corr2) + a.eps);
  }
}
__device__ __forceinline__ void ddp_update4(const DdpBucketArgs& a, float4& pm, const float4& g, float4& m, float4& v) {
  ddp_update1(a, pm.x, g.x, m.x, v.x);
  ddp_update1(a, pm.y, g.y, m.y, v.y);
  ddp_update1(a, pm.z, g.z, m.z, v.z);
  ddp_update1(a, pm.w, g.w, m.w, v.w);
}

// WT = compile-time world size (1, 2, 4, 8) or 0 for "read it from the arguments".  Each thread
// handles G = 8 / WT groups of 4 elements per trip and issues the G x W peer loads before it
// consumes any, i.e. 8 sixteen-byte loads in flight per thread whatever the world size.
// NVLS = the gradient / parameter buffers are also mapped through a multicast object: the G loads per
// trip are switch-side reductions over all ranks and the zero / parameter stores go out once.
template <int WT, bool NVLS>
__global__ void __launch_bounds__(256, 2) ddp_bucket_step_kernel(const DdpBucketArgs a) {
  const int W = WT > 0 ? WT : a.world;
  const int R = a.rank;
  constexpr int G = NVLS ? 8 : (WT > 0 ? 8 / WT : 1);
  constexpr int WMAX = NVLS ? 1 : (WT > 0 ? WT : RT_MAX_PEERS);
  int* my_flags = a.flags[R];
  // ---- start barrier: tell every peer this rank's bucket gradients are final, wait for theirs.  A CTA whose
  // wait runs out skips the data phase but still takes part in the end protocol below, so the completion
  // counter is back at zero for the next launch whatever happened.
  bool ok = true;
  if (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x < W && int(threadIdx.x) != R) {
      __threadfence_system();
      st_release_sys(a.flags[threadIdx.x] + a.start_slot + R, a.epoch);
    }
    ok = wait_flags(my_flags + a.start_slot, W, R, a.epoch, a.timeout_ns, a.status);
  }

  const long long base = a.bucket_start + (long long)R * a.chunk_len;  // flat index of my shard
  const long long n4 = ok ? (a.chunk_len >> 2) : 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool has_m = a.m != nullptr, has_v = a.v != nullptr;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += G * stride) {
    float4 v[G][WMAX];
    long long e[G];
    bool on[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long i = i0 + g * stride;
      on[g] = i < n4;
      e[g] = base + ((on[g] ? i : i0) << 2);
      if (NVLS) {
        if (on[g]) v[g][0] = mc_ld_reduce_f4(a.mc_grad + e[g]);
      } else {
#pragma unroll
        for (int p = 0; p < WMAX; ++p)
          if (p < W && on[g]) v[g][p] = ld_peer_f4(a.grad[p] + e[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!on[g]) continue;
      float4 sum;
      // Gradients are zeroed for the next backward pass: this rank's copy here, the peers' copies by their owners
      // after the end-of-step wait (a local memset instead of N - 1 remote stores per element).
      if (NVLS) {
        sum = v[g][0];
      } else {
        sum = z;
#pragma unroll
        for (int p = 0; p < WMAX; ++p) {
          if (p < W) {
            sum.x += v[g][p].x; sum.y += v[g][p].y; sum.z += v[g][p].z; sum.w += v[g][p].w;
          }
        }
      }
      // This rank's copy of its own slice is zeroed here on the peer-load path (same address as the load above, so
      // the hardware orders the two).  On the multimem path the switch reads this copy through ANOTHER virtual
      // address; a zero stored from the same kernel, even one computed from the loaded value, was measured to make
      // this rank's own gradient read as zero in the reduction.  There the whole buffer is cleared by its owner
      // after the end-of-step wait instead.
      if (!NVLS) *reinterpret_cast<float4*>(a.grad[R] + e[g]) = z;
      float4 pm = *reinterpret_cast<float4*>(a.master + e[g]);
      float4 m = has_m ? *reinterpret_cast<float4*>(a.m + e[g]) : z;
      float4 vv = has_v ? *reinterpret_cast<float4*>(a.v + e[g]) : z;
      ddp_update4(a, pm, sum, m, vv);
      *reinterpret_cast<float4*>(a.master + e[g]) = pm;
      if (has_m) *reinterpret_cast<float4*>(a.m + e[g]) = m;
      if (has_v) *reinterpret_cast<float4*>(a.v + e[g]) = vv;
      uint2 w;
      w.x = pack_bf16x2(pm.x, pm.y);
      w.y = pack_bf16x2(pm.z, pm.w);
      if (NVLS) {
        mc_st_b32x2(reinterpret_cast<__nv_bfloat16*>(a.mc_lp) + e[g], w.x, w.y);
      } else {
#pragma unroll
        for (int p = 0; p < WMAX; ++p)
          if (p < W) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.lp[p]) + e[g]) = w;
      }
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

void ddp_bucket_step(const DdpBucketArgs& a, int n_ctas, cudaStream_t stream) {
  RT_CHECK(a.world >= 1 && a.world <= RT_MAX_PEERS, "ddp: world size must be in [1, 8]");
  RT_CHECK(a.chunk_len % 4 == 0 && a.bucket_start % 4 == 0, "ddp: bucket geometry must be 4-aligned");
  RT_CHECK(a.opt_mode == OPT_ADAMW || a.opt_mode == OPT_ADAM || a.opt_mode == OPT_SGD, "ddp: optimizer must be AdamW, Adam or SGD");
  RT_CHECK(a.opt_mode == OPT_SGD || (a.m != nullptr && a.v != nullptr), "ddp: Adam / AdamW need both moment buffers");
  RT_CHECK(a.opt_mode != OPT_SGD || a.beta1 == 0.f || a.m != nullptr, "ddp: SGD with momentum needs its buffer");
  if (a.chunk_len == 0) return;
  if (n_ctas <= 0) n_ctas = 2 * sm_count(current_device());
  const bool nvls = a.world > 1 && a.mc_grad != nullptr && a.mc_lp != nullptr;
  if (nvls) {
    ddp_bucket_step_kernel<0, true><<<n_ctas, 256, 0, stream>>>(a);
  } else {
    switch (a.world) {
      case 1: ddp_bucket_step_kernel<1, false><<<n_ctas, 256, 0, stream>>>(a); break;
      case 2: ddp_bucket_step_kernel<2, false><<<n_ctas, 256, 0, stream>>>(a); break;
      case 4: ddp_bucket_step_kernel<4, false><<<n_ctas, 256, 0, stream>>>(a); break;
      case 8: ddp_bucket_step_kernel<8, false><<<n_ctas, 256, 0, stream>>>(a); break;
      default: ddp_bucket_step_kernel<0, false><<<n_ctas, 256, 0, stream>>>(a); break;
    }
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
