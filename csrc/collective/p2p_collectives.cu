// Collectives over NVLink peer memory (symmetric buffers): all-reduce (one-shot and two-shot), all-gather,
// reduce-scatter, broadcast.  One kernel per call; every rank launches the same kernel on its own GPU.
//
//   one-shot all-reduce  every rank reads all W inputs and sums them (W x traffic, one flag round: for small
//                        messages such as tensor-parallel decode activations, where latency is everything)
//   two-shot all-reduce  rank r sums chunk r of all inputs into its result buffer, publishes it, then gathers
//                        the other chunks (2 x (W-1)/W traffic: for large messages)
//   all-gather / reduce-scatter / broadcast: the pull halves of the above.
//
// Protocol (flags are int32 words in symmetric memory, values are call epochs, so nothing is ever reset):
//   ready[r]   set on every peer by rank r at kernel start: "my input buffer holds this call's data"
//   stage2[r]  (two-shot) set on every peer when rank r's reduced chunk is in its result buffer
//   done[r]    set on every peer when rank r will not read peer memory again in this call; CTA 0 of every rank
//              waits for all of them before the kernel ends, so a buffer can be overwritten right after.
// Peer data is read with ld.global.cg 16-byte loads (W of them in flight per thread), sums are fp32.
// All waits are bounded (globaltimer deadline -> status word, then the CTA leaves).  The grid never exceeds
// two CTAs per SM, so all CTAs are resident and the in-kernel grid barrier (two words of local memory) is safe.
// The call epoch is a device word the kernel advances itself, so the launch can be replayed from a CUDA graph.
//
// These replace the reference's host-side "collectives" (ring / tree / host-staged loops over Vec<f32>,
// src/gpu/multi_gpu.rs:583-940) and the no-op NCCL shells (src/distributed/nccl_integration.rs:75-144).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace rt {

namespace {

__device__ __forceinline__ void pc_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int pc_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 pc_ld_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename T> struct PV { static constexpr int N = 8; };
template <> struct PV<float> { static constexpr int N = 4; };
__device__ __forceinline__ float pcf(float v) { return v; }
__device__ __forceinline__ float pcf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float pcf(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T pct(float v);
template <> __device__ __forceinline__ float pct<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 pct<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half pct<__half>(float v) { return __float2half(v); }

// Thread `which` of the CTA waits for flags[which] >= epoch (which < n, which != skip); CTA-wide verdict.
__device__ __forceinline__ bool pc_wait_all(const int* flags, int n, int skip, int epoch, unsigned long long timeout_ns,
                                            int* status) {
  bool ok = true;
  if ((int)threadIdx.x < n && (int)threadIdx.x != skip) {
    const int* f = flags + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    unsigned it = 0;
    while (pc_ld_acquire_sys(f) < epoch) {
      if ((++it & 0x3ff) == 0 && globaltimer_ns() - t0 > timeout_ns) {
        atomicCAS(status, 0, RT_ERR_TIMEOUT_PEER);
        ok = false;
        break;
      }
      __nanosleep(32);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Grid barrier: state[0] counts arrivals and is reset by the last arriver, state[1] is a generation word that only
// grows; `gen` must be larger than in any earlier barrier on this state (2 * epoch - 1 and 2 * epoch here).
__device__ __forceinline__ bool pc_grid_barrier(unsigned* state, unsigned gen, unsigned long long timeout_ns, int* status) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned old = atomicAdd(&state[0], 1u);
    if (old == gridDim.x - 1) {
      state[0] = 0;
      __threadfence();
      atomicExch(&state[1], gen);
    } else {
      const unsigned long long t0 = globaltimer_ns();
      unsigned it = 0;
      while (*reinterpret_cast<volatile unsigned*>(&state[1]) < gen) {
        if ((++it & 0x3ff) == 0 && globaltimer_ns() - t0 > timeout_ns) {
          atomicCAS(status, 0, RT_ERR_TIMEOUT_PEER);
          ok = false;
          break;
        }
        __nanosleep(32);
      }
    }
    __threadfence();
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// out[i] = sum_r in_r[off + i], i in [0, n) (vectors of 16 bytes); `in` are peer pointers.
template <typename T>
__device__ __forceinline__ void pc_reduce_range(const P2PCollArgs& a, const T* const* in, T* out, long long off, long long n) {
  constexpr int V = PV<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    uint4 raw[RT_MAX_PEERS];
#pragma unroll
    for (int r = 0; r < RT_MAX_PEERS; ++r)
      if (r < a.world) raw[r] = pc_ld_cg(in[r] + off + i * V);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
    for (int r = 0; r < RT_MAX_PEERS; ++r)
      if (r < a.world) {
        const T* v = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += pcf(v[e]);
      }
    uint4 w;
    T* o = reinterpret_cast<T*>(&w);
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = pct<T>(acc[e]);
    *reinterpret_cast<uint4*>(out + i * V) = w;
  }
}

template <typename T>
__device__ __forceinline__ void pc_copy_range(const T* src, T* dst, long long n) {
  constexpr int V = PV<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride)
    *reinterpret_cast<uint4*>(dst + i * V) = pc_ld_cg(src + i * V);
}

template <typename T>
__global__ void __launch_bounds__(256, 2) p2p_collective_kernel(const P2PCollArgs a) {
  const int W = a.world, R = a.rank;
  int* my_flags = a.flags[R];
  const T* in[RT_MAX_PEERS];
  T* res[RT_MAX_PEERS];
  for (int r = 0; r < RT_MAX_PEERS; ++r) {
    in[r] = reinterpret_cast<const T*>(a.in[r < W ? r : 0]);
    res[r] = reinterpret_cast<T*>(a.result[r < W ? r : 0]);
  }
  T* out = reinterpret_cast<T*>(a.out);
  bool ok = true;
  // The call epoch lives in device memory (read here, advanced by CTA 0 after the last barrier), so a captured
  // CUDA graph can replay this kernel: nothing call-specific is baked into the launch.
  const int epoch = *reinterpret_cast<volatile int*>(a.epoch_dev) + 1;
  // ---- everyone's input is in place
  if (W > 1) {
    if (blockIdx.x == 0 && (int)threadIdx.x < W && (int)threadIdx.x != R) {
      __threadfence_system();
      pc_st_release_sys(a.flags[threadIdx.x] + R, epoch);
    }
    ok = pc_wait_all(my_flags, W, R, epoch, a.timeout_ns, a.status);
  }
  if (ok) {
    const long long n = a.numel;
    if (a.mode == P2P_ALL_REDUCE_ONE_SHOT) {
      pc_reduce_range<T>(a, in, out, 0, n);
    } else if (a.mode == P2P_REDUCE_SCATTER) {
      pc_reduce_range<T>(a, in, out, (long long)R * (n / W), n / W);
    } else if (a.mode == P2P_ALL_GATHER) {
      for (int s = 0; s < W; ++s) {
        const int r = (R + s) % W;
        pc_copy_range<T>(in[r], out + (long long)r * n, n);
      }
    } else if (a.mode == P2P_BROADCAST) {
      pc_copy_range<T>(in[a.root], out, n);
    } else {  // two-shot all-reduce
      const long long chunk = n / W;
      pc_reduce_range<T>(a, in, res[R] + (long long)R * chunk, (long long)R * chunk, chunk);
      // all CTAs of this rank have written their part of the chunk -> publish it
      ok = pc_grid_barrier(a.grid_counter, 2u * (unsigned)epoch - 1u, a.timeout_ns, a.status);
      if (ok && W > 1) {
        if (blockIdx.x == 0 && (int)threadIdx.x < W && (int)threadIdx.x != R) {
          __threadfence_system();
          pc_st_release_sys(a.flags[threadIdx.x] + W + R, epoch);
        }
        ok = pc_wait_all(my_flags + W, W, R, epoch, a.timeout_ns, a.status);
      }
      if (ok) {
        for (int s = 0; s < W; ++s) {
          const int r = (R + s) % W;
          pc_copy_range<T>(res[r] + (long long)r * chunk, out + (long long)r * chunk, chunk);
        }
      }
    }
  }
  // ---- nobody reads peer memory any more: say so, hold the kernel until all peers have said it, advance the epoch
  const bool ok2 = pc_grid_barrier(a.grid_counter, 2u * (unsigned)epoch, a.timeout_ns, a.status);
  if (blockIdx.x == 0) {
    if (W > 1) {
      if (ok && ok2 && (int)threadIdx.x < W && (int)threadIdx.x != R) pc_st_release_sys(a.flags[threadIdx.x] + 2 * W + R, epoch);
      pc_wait_all(my_flags + 2 * W, W, R, epoch, a.timeout_ns, a.status);
    }
    if (threadIdx.x == 0) *a.epoch_dev = epoch;
  }
}

}  // namespace

void p2p_collective(const P2PCollArgs& a, cudaStream_t stream) {
  RT_CHECK(a.world >= 1 && a.world <= RT_MAX_PEERS && a.rank >= 0 && a.rank < a.world, "p2p_collective: bad world / rank");
  RT_CHECK(a.mode >= P2P_ALL_REDUCE_ONE_SHOT && a.mode <= P2P_BROADCAST, "p2p_collective: unknown mode");
  RT_CHECK(a.dtype >= DT_F32 && a.dtype <= DT_F16, "p2p_collective: dtype must be fp32, bf16 or fp16");
  RT_CHECK(a.epoch_dev != nullptr && a.grid_counter != nullptr, "p2p_collective: device epoch word and barrier state required");
  const int vec = a.dtype == DT_F32 ? 4 : 8;
  const long long unit = (a.mode == P2P_ALL_REDUCE_TWO_SHOT || a.mode == P2P_REDUCE_SCATTER) ? (long long)vec * a.world : vec;
  RT_CHECK(a.numel % unit == 0, "p2p_collective: element count must be a multiple of the 16-byte vector (times the world size "
                                "for reduce-scatter / two-shot all-reduce)");
  if (a.numel == 0) return;
  const int device = current_device();
  const long long nvec = a.numel / vec;
  const int grid = (int)std::max<long long>(1, std::min<long long>((nvec + 255) / 256, 2LL * sm_count(device)));
  P2PCollArgs b = a;
  b.status = status_word(device);
  if (a.dtype == DT_F32) p2p_collective_kernel<float><<<grid, 256, 0, stream>>>(b);
  else if (a.dtype == DT_BF16) p2p_collective_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(b);
  else p2p_collective_kernel<__half><<<grid, 256, 0, stream>>>(b);
  RT_LAUNCH_CHECK();
}

}  // namespace rt
