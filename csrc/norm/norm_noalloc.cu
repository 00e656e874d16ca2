// See norm_noalloc.h: LayerNorm / RMSNorm backward with its partial-sum scratch in a fixed
// device array instead of caller- or allocator-provided memory.
#include "norm_noalloc.h"

#include <atomic>
#include <string>

#include "../api.h"
#include "../common/launch.h"

namespace {

// Scratch for the two-stage d(gamma)/d(beta) reduction: [2][n_partial][C] floats.
static __device__ __align__(256) float g_norm_scratch[RT_NORM_NOALLOC_SCRATCH_FLOATS];

// Device address of g_norm_scratch per device.  In host code the name g_norm_scratch is only a
// handle for the runtime, not a device pointer, so it must be translated once per device.
// Two host threads may make the first call on one device at the same time: both resolve the same
// values, the SM count is stored first and the address last with release order, and readers load
// the address with acquire order, so whoever sees a non-null address also sees the SM count.
constexpr int kMaxDevices = 64;
std::atomic<float*> g_scratch_addr[kMaxDevices];
std::atomic<int> g_sm_count[kMaxDevices];
thread_local std::string g_last_error;

int fail_with(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

}  // namespace

extern "C" const char* rt_noalloc_last_error(void) { return g_last_error.c_str(); }

extern "C" int rt_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma,
                                   const float* mean, const float* rstd, const void* dres,
                                   void* dx, float* dgamma, float* dbeta, long long rows, int C,
                                   int rms, void* stream) {
  g_last_error.clear();
  if (C <= 0 || C % 8 != 0 || C > RT_NORM_NOALLOC_MAX_C || rows < 0)
    return fail_with(RT_NOALLOC_ERR_SIZE,
                     "rt_norm_bwd_noalloc: feature size " + std::to_string(C) +
                         " not supported (multiple of 8, at most " +
                         std::to_string(RT_NORM_NOALLOC_MAX_C) + ") or negative row count");
  if (rows == 0) return RT_NOALLOC_OK;
  if (!dy || !x || !gamma || !rstd || !dx || (!rms && !mean))
    return fail_with(RT_NOALLOC_ERR_ARG, "rt_norm_bwd_noalloc: null input/output pointer");

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return fail_with(RT_NOALLOC_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices)
    return fail_with(RT_NOALLOC_ERR_ARG, "rt_norm_bwd_noalloc: device index " + std::to_string(device) +
                                             " is outside the supported range [0, " + std::to_string(kMaxDevices) + ")");
  float* scratch = g_scratch_addr[device].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // One-time set-up for this device (current right now): translate the symbol to its address.
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_norm_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail_with(RT_NOALLOC_ERR_CUDA,
                       std::string("cudaGetSymbolAddress(g_norm_scratch): ") + cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess || sms <= 0)
      return fail_with(RT_NOALLOC_ERR_CUDA,
                       std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
    g_sm_count[device].store(sms, std::memory_order_relaxed);
    g_scratch_addr[device].store(ptr, std::memory_order_release);
    scratch = ptr;
  }

  rt::NormArgs a{};
  a.dy = dy;
  a.x = x;
  a.gamma = gamma;
  a.mean = const_cast<float*>(mean);
  a.rstd = const_cast<float*>(rstd);
  a.dres = dres;
  a.dx = dx;
  a.dgamma = dgamma;
  a.dbeta = rms ? nullptr : dbeta;
  a.rows = rows;
  a.C = C;
  a.rms = rms != 0;
  // as many partial-sum rows as the normal path would use, capped by the fixed array
  const int fit = RT_NORM_NOALLOC_SCRATCH_FLOATS / (2 * C);
  a.n_partial = std::min(rt::norm_bwd_num_partials(rows, g_sm_count[device].load(std::memory_order_relaxed)), fit);
  a.partial = scratch;
  try {
    rt::norm_bwd(a, static_cast<cudaStream_t>(stream));
  } catch (const std::exception& ex) {
    return fail_with(RT_NOALLOC_ERR_CUDA, ex.what());
  }
  return RT_NOALLOC_OK;
}
