// Host-side helpers shared by every launcher.  Torch-free on purpose: kernel translation
// units include only this and compile in seconds; the tensor-facing glue lives in
// csrc/bindings.cpp.
#pragma once
#include <utility>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace rt {

// Number of kernels launched by this library since process start.
long long launch_count();
void count_launch(int n = 1);
bool bounds_check_build();  // compiled with -DRT_BOUNDS_CHECK

// One int32 status word per device, zero while healthy.  Kernels CAS an error code into
// it when a bounded wait expires (see ptx.cuh); read_status() synchronises the device and
// returns + clears it.
int* status_word(int device);
int read_status(int device);

int current_device();
int sm_count(int device);

[[noreturn]] void fail(const std::string& msg);

#define RT_CHECK(cond, msg)                                       \
  do {                                                            \
    if (!(cond)) ::rt::fail(std::string("rustorch_b200: ") + msg); \
  } while (0)

#define RT_CUDA_CHECK(expr)                                                               \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      ::rt::fail(std::string(#expr) + " failed: " + cudaGetErrorString(_e));              \
  } while (0)

#define RT_LAUNCH_CHECK()                                                                 \
  do {                                                                                    \
    cudaError_t _e = cudaGetLastError();                                                  \
    if (_e != cudaSuccess)                                                                \
      ::rt::fail(std::string("kernel launch failed: ") + cudaGetErrorString(_e));         \
    ::rt::count_launch();                                                                 \
  } while (0)

// Tiled 2-byte-element tensor map over a [d2][d1][d0] array (d0 contiguous) with a
// 128-byte swizzle.  Strides in elements.  box = {b0, b1, 1}.
CUtensorMap make_tmap_2byte(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                            uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0,
                            uint32_t b1);
// Rank-4 variant: [d3][d2][d1][d0], box = {b0, b1, 1, 1}.
CUtensorMap make_tmap_2byte_4d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0,
                               uint32_t b1);
// Rank-4 fp32 map [d3][d2][d1][d0] (strides in elements) with the 128-byte swizzle: box = 32 floats x b1 rows.  Used for
// TMA reduce-add (cp.reduce.async.bulk.tensor ... .add) of fp32 tiles staged in shared memory.
CUtensorMap make_tmap_f32_4d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2,
                             uint64_t s3, uint32_t b0, uint32_t b1);
// Plain (unswizzled) rank-2 map over rows of `row_bytes` bytes seen as 32-bit words (elem_bytes = 4) or
// 16-bit values (elem_bytes = 2): dims {row_elems, rows}, box {box_elems, box_rows}; out-of-range parts of a
// box read as zero.  row_bytes must be a multiple of 16.
CUtensorMap make_tmap_rows(const void* base, int elem_bytes, uint64_t row_elems, uint64_t rows,
                           uint32_t box_elems, uint32_t box_rows);
// Rank-2 map over byte rows seen as 32-bit words with the 128-byte swizzle: box = 128 bytes x box_rows rows; row r of
// a box lands at r * 128 with its 16-byte chunk c stored at chunk position c ^ (r & 7).
CUtensorMap make_tmap_words_sw128(const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows);
// Rank-4 map over a channels-last activation tensor [N][H][W][C] (2-byte elements, C contiguous, 128-byte swizzle):
// a box covers 64 channels x box_w x box_h x box_n positions taken every `stride` pixels along W and H.
CUtensorMap make_tmap_nhwc(const void* base, uint64_t C, uint64_t W, uint64_t H, uint64_t N, uint32_t box_w, uint32_t box_h,
                           uint32_t box_n, uint32_t stride);

// True unless RUSTORCH_PDL=0: kernels of the decode path are then launched with programmatic stream serialization
// (the next kernel's prologue and weight prefetch overlap the tail of the previous one; see pdl_wait in ptx.cuh).
bool pdl_enabled();

#ifdef __CUDACC__
// kern<<<grid, block, smem, stream>>>(args...) with the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...));
}
#endif

}  // namespace rt
