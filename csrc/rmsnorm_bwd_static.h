// RMSNorm backward that allocates nothing: for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework. It exists for callers that sit
// where an allocation is not allowed or not wanted: a C or C++ host that links this library without
// PyTorch and so has no caching allocator to ask for a workspace; code that runs while another
// component owns all remaining device memory (a sampler that was given the whole free pool for its
// KV cache); and latency-critical loops in which a cudaMalloc or cudaFree, which synchronise the
// device, must never happen. The regular entry point, axb_rmsnorm_bwd, leaves the workspace to its
// caller; this one brings its own.
//
// The workspace is a fixed array in the library's device image, AXB_RMSNORM_BWD_STATIC_MAX_FLOATS
// floats (9.25 MiB) per device. It holds the per-block partial sums of the weight gradient:
// axb_rmsnorm_bwd_partials(T) rows of H floats. A call whose partials do not fit (rows * H above the
// maximum) is refused with AXB_LAUNCH_TOO_LARGE and launches nothing. The row count is
// min(T, 4 x the SM count of the device this process first used), i.e. at most 592 on a 148-SM B200:
// there the maximum covers hidden sizes up to 4096 at any token count, and larger hidden sizes while
// T < MAX_FLOATS / H. On a part with more SMs the row cap is higher, so hidden 4096 is refused once
// T exceeds MAX_FLOATS / 4096 = 592 rows; the limit itself never changes.
// axb_rmsnorm_bwd_static_error() gives the text for the last refusal on the calling thread.
//
// Set-up: the first call on each device (with that device current) looks up the array's address
// with cudaGetSymbolAddress and keeps it; the library calls no allocating routine, then or later.
// Make that first call, or axb_rmsnorm_bwd_static_setup(), before any stream capture begins.
// Several host threads may make the first call on a device at once: each stores the same address,
// so the unsynchronised write is harmless. The stream passed in must belong to the current device
// (a null stream always does); a stream of another device is refused with AXB_LAUNCH_BAD_ARG.
// Nothing in the workspace has to start at zero: each call writes every partial it later reads.
//
// One workspace per device means that two calls on the same device whose kernels can overlap
// (different streams, or different host threads on different streams) race on it and give wrong
// weight gradients. Calls on one stream are ordered and safe.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define AXB_RMSNORM_BWD_STATIC_MAX_FLOATS (592 * 4096)

// Looks up the workspace of the current device. 0 on success, AXB_LAUNCH_CUDA_ERROR otherwise.
int axb_rmsnorm_bwd_static_setup(void);

// Same arguments and results as axb_rmsnorm_bwd, without the scratch pointer:
//   dx[T,H] (bf16) = dres + d rmsnorm / dx ;  dw[H] (fp32) (+)= sum_t dy * xhat.
// dres may be null. Returns 0, or a negative AXB_LAUNCH_* code.
int axb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                           const void* dres, void* dx, float* dw, int dw_accumulate, long long T,
                           int H, void* stream);

// Text of the last error of the two calls above on this thread ("" when there was none).
const char* axb_rmsnorm_bwd_static_error(void);

#ifdef __cplusplus
}
#endif
