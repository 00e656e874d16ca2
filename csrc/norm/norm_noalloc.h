// Allocation-free C entry point for the LayerNorm / RMSNorm backward pass.
//
// This entry point has no counterpart in the reference (RusTorch); it exists for callers of
// this library that are not allowed to allocate device memory at the moment they need the
// kernel: code running inside a memory-pool callback or between the begin/end of a stream
// capture, real-time inference loops that forbid allocator calls after warm-up, and plain C
// hosts that link the shared object without torch's caching allocator behind them.
//
// The normal path (rt::norm_bwd, reached from Python through `_C.norm_bwd`) receives a scratch
// buffer for the per-CTA partial sums of d(gamma)/d(beta) that the tensor glue allocates with
// torch.  Here the same kernels run with that scratch placed in a fixed array in device
// global memory that is part of the library image, so the call itself performs no cudaMalloc,
// cudaFree or any other allocating routine.
//
// Limits and rules
//  * feature size C: a multiple of 8, at most RT_NORM_NOALLOC_MAX_C (8192); larger sizes are
//    rejected with RT_NOALLOC_ERR_SIZE.  `rows` is unlimited (the number of partial-sum rows is
//    capped to what fits the array).
//  * the array holds RT_NORM_NOALLOC_SCRATCH_FLOATS floats (4 MiB) and every GPU that loads the
//    library keeps it until the process exits.
//  * the first call on a device looks up the device address of the array (one
//    cudaGetSymbolAddress, no allocation).  Make that first call before starting any stream
//    capture on that device.  The per-device cache of that address is published with
//    release / acquire atomics, so host threads may make their first calls concurrently.
//  * devices with an index of 64 or more are rejected with RT_NOALLOC_ERR_ARG.
//  * all calls on a device share the one array.  It keeps whatever the previous call left in
//    it; nothing in it needs to start at zero because the first kernel overwrites every
//    partial-sum row the second kernel reads.  Two calls whose kernels overlap on the GPU
//    (different streams without an ordering between them) race on the array: serialise them.
//  * dgamma / dbeta are accumulated into (+=), exactly like the allocating path.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RT_NORM_NOALLOC_MAX_C 8192
#define RT_NORM_NOALLOC_SCRATCH_FLOATS (1 << 20)

#define RT_NOALLOC_OK 0
#define RT_NOALLOC_ERR_SIZE (-1)    /* C above the maximum, not a multiple of 8, or rows < 0 */
#define RT_NOALLOC_ERR_ARG (-2)     /* a required pointer is null, or the device index is 64 or more */
#define RT_NOALLOC_ERR_CUDA (-3)    /* a CUDA call failed; see rt_noalloc_last_error() */

// dy, x, dres (optional), dx: bf16 [rows][C]; gamma: bf16 [C]; mean (LayerNorm only), rstd:
// fp32 [rows] as saved by the forward pass; dgamma / dbeta: fp32 [C] or null.  `rms` != 0
// selects RMSNorm (mean and dbeta ignored).  `stream` is a cudaStream_t (null = default stream).
// The device that owns the buffers must be current.  Returns RT_NOALLOC_OK or an error code.
int rt_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                        const float* rstd, const void* dres, void* dx, float* dgamma,
                        float* dbeta, long long rows, int C, int rms, void* stream);

// Text of the last error reported by rt_norm_bwd_noalloc on the calling thread ("" if none).
const char* rt_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
