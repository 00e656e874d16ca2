#include "launch.h"

#include <cstdlib>

#include <atomic>
#include <mutex>
#include <unordered_map>

namespace rt {

namespace {
std::atomic<long long> g_launches{0};
std::mutex g_mu;
int* g_status[64] = {nullptr};
int g_sms[64] = {0};

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread.
// Threads that have only ever queried the device (e.g. autograd's backward threads) may not
// have the primary context bound yet; a no-op runtime call binds it.
void bind_context_once() {
  static thread_local bool bound = false;
  if (!bound) {
    RT_CUDA_CHECK(cudaFree(nullptr));
    bound = true;
  }
}

EncodeFn encode_fn() {
  bind_context_once();
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    RT_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    RT_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess,
             "cuTensorMapEncodeTiled not available from the driver");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}
}  // namespace

void fail(const std::string& msg) { throw std::runtime_error(msg); }

long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
bool bounds_check_build() {
#ifdef RT_BOUNDS_CHECK
  return true;
#else
  return false;
#endif
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int current_device() {
  int d = 0;
  RT_CUDA_CHECK(cudaGetDevice(&d));
  return d;
}

int sm_count(int device) {
  if (g_sms[device] == 0) {
    int v = 0;
    RT_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
    g_sms[device] = v;
  }
  return g_sms[device];
}

int* status_word(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[device]) {
    int prev = current_device();
    RT_CUDA_CHECK(cudaSetDevice(device));
    int* p = nullptr;
    RT_CUDA_CHECK(cudaMalloc(&p, sizeof(int) * 16));
    RT_CUDA_CHECK(cudaMemset(p, 0, sizeof(int) * 16));
    RT_CUDA_CHECK(cudaSetDevice(prev));
    g_status[device] = p;
  }
  return g_status[device];
}

int read_status(int device) {
  int* p = status_word(device);
  int prev = current_device();
  RT_CUDA_CHECK(cudaSetDevice(device));
  int v = 0;
  RT_CUDA_CHECK(cudaDeviceSynchronize());
  RT_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) RT_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
  RT_CUDA_CHECK(cudaSetDevice(prev));
  return v;
}

namespace {
// A tensor map is a pure function of (base, extents, strides, box): the maps of one training or decode step recur every
// step because the caching allocator hands the same addresses out again, so they are kept per host thread instead of
// being encoded by the driver on every launch.
struct TmapKey {
  const void* base;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1;
  bool operator==(const TmapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 && b1 == o.b1;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    for (uint64_t v : {k.d0, k.d1, k.d2, k.s1, k.s2, (uint64_t(k.b0) << 32) | k.b1}) h = (h ^ v) * 0x100000001B3ull + (h >> 29);
    return size_t(h);
  }
};
CUtensorMap encode_tmap_2byte(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                              uint64_t stride2_elems, uint32_t b0, uint32_t b1);
}  // namespace

CUtensorMap make_tmap_2byte(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                            uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0,
                            uint32_t b1) {
  thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{base, d0, d1, d2, stride1_elems, stride2_elems, b0, b1};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() >= 8192) cache.clear();
  const CUtensorMap m = encode_tmap_2byte(base, d0, d1, d2, stride1_elems, stride2_elems, b0, b1);
  cache.emplace(key, m);
  return m;
}

namespace {
CUtensorMap encode_tmap_2byte(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0,
                              uint32_t b1) {
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RT_CHECK((stride1_elems * 2) % 16 == 0,
           "TMA row stride must be a multiple of 16 bytes (got " + std::to_string(stride1_elems) +
               " elements)");
  RT_CHECK(d2 == 1 || (stride2_elems * 2) % 16 == 0,
           "TMA batch stride must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, (d2 == 1 ? stride1_elems * d1 : stride2_elems) * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS,
           "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)) + " dims=" +
               std::to_string(d0) + "," + std::to_string(d1) + "," + std::to_string(d2) +
               " strides=" + std::to_string(strides[0]) + "," + std::to_string(strides[1]) +
               " box=" + std::to_string(b0) + "," + std::to_string(b1));
  return m;
}
}  // namespace

CUtensorMap make_tmap_2byte_4d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0,
                               uint32_t b1) {
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RT_CHECK((s1 * 2) % 16 == 0 && (s2 * 2) % 16 == 0 && (s3 * 2) % 16 == 0,
           "TMA strides must be multiples of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1 * 2, s2 * 2, s3 * 2};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS,
           "cuTensorMapEncodeTiled(4d) failed with code " + std::to_string(int(r)));
  return m;
}

CUtensorMap make_tmap_rows(const void* base, int elem_bytes, uint64_t row_elems, uint64_t rows,
                           uint32_t box_elems, uint32_t box_rows) {
  RT_CHECK(elem_bytes == 2 || elem_bytes == 4, "make_tmap_rows: 2- or 4-byte elements");
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RT_CHECK((row_elems * elem_bytes) % 16 == 0, "TMA row pitch must be a multiple of 16 bytes");
  RT_CHECK(box_elems <= 256 && box_rows <= 256 && (box_elems * elem_bytes) % 16 == 0, "TMA box out of range");
  CUtensorMap m;
  cuuint64_t dims[2] = {row_elems, rows};
  cuuint64_t strides[1] = {row_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_elems, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(&m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                           const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(rows) failed with code " + std::to_string(int(r)));
  return m;
}

CUtensorMap make_tmap_words_sw128(const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0 && row_bytes % 16 == 0, "TMA rows must be 16-byte aligned");
  RT_CHECK(box_rows >= 1 && box_rows <= 256, "TMA box out of range");
  CUtensorMap m;
  cuuint64_t dims[2] = {row_bytes / 4, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(words, sw128) failed with code " + std::to_string(int(r)));
  return m;
}

CUtensorMap make_tmap_f32_4d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                             uint64_t s3, uint32_t b0, uint32_t b1) {
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RT_CHECK((s1 * 4) % 16 == 0 && (s2 * 4) % 16 == 0 && (s3 * 4) % 16 == 0, "TMA strides must be multiples of 16 bytes");
  RT_CHECK(b0 * 4 == 128 && b1 >= 1 && b1 <= 256, "fp32 swizzled TMA box: 32 elements (128 bytes) wide, at most 256 rows");
  CUtensorMap m;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1 * 4, s2 * 4, s3 * 4};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(f32 4d) failed with code " + std::to_string(int(r)));
  return m;
}

CUtensorMap make_tmap_nhwc(const void* base, uint64_t C, uint64_t W, uint64_t H, uint64_t N, uint32_t box_w, uint32_t box_h,
                           uint32_t box_n, uint32_t stride) {
  RT_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RT_CHECK(C % 8 == 0, "channels-last TMA needs a multiple of 8 channels");
  RT_CHECK(box_w * stride <= 256 && box_h * stride <= 256 && box_n <= 256 && stride >= 1 && stride <= 8, "TMA box out of range");
  CUtensorMap m;
  cuuint64_t dims[4] = {C, W, H, N};
  cuuint64_t strides[3] = {C * 2, W * C * 2, H * W * C * 2};
  cuuint32_t box[4] = {64, box_w * stride, box_h * stride, box_n};  // extent in the tensor; every stride-th element is taken
  cuuint32_t estr[4] = {1, stride, stride, 1};
  if (stride > 1) {  // the extent only has to reach the last element taken
    box[1] = (box_w - 1) * stride + 1;
    box[2] = (box_h - 1) * stride + 1;
  }
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(nhwc) failed with code " + std::to_string(int(r)));
  return m;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("RUSTORCH_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace rt
