// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation.  It exists for
// code that runs where cudaMalloc (and any allocating library call, torch's caching
// allocator included) is off limits: a real-time serving loop whose memory budget was
// fixed at start-up, a plugin inside a host process that owns the GPU heap, or any place
// where an allocation could fail or stall at a bad moment.  Such callers hand in every
// input and output buffer themselves; the only extra memory the computation needs, the
// per-block partial sums of the weight gradient, lives in a fixed array inside this
// library.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats (8 MiB per GPU that loads the library,
// held until the process exits).  A call needs ceil(rows / 32) * width floats.
#define AGB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

// dx[rows, width] (bf16) and dw[width] (fp32) of y = w * rms_norm(x), given grad = dL/dy.
//   grad, x, dx : bf16 [rows, width]      w : bf16 [width]
//   rstd        : fp32 [rows], 1/sqrt(mean(x^2) + eps) as saved by the forward pass
//   dw          : fp32 [width], overwritten
//   stream      : a cudaStream_t (may be null for the default stream)
// All pointers are device pointers supplied by the caller, on the current device.
//
// Limits: width a multiple of 8 and at most 8192; ceil(rows / 32) * width must not exceed
// AGB_NOALLOC_SCRATCH_FLOATS.  A request beyond that is refused with a negative return
// value and a message (see agb_noalloc_last_error); nothing is launched.
//
// The first call on a device looks up the device address of the scratch array.  Make that
// first call before starting any stream capture on that device.
//
// Every call on a device uses the same scratch array, which keeps whatever the previous
// call left in it.  The part a call reads is fully rewritten by that call first, so no
// clearing is needed, but two calls whose kernels may overlap on the GPU (different
// streams without an ordering between them) would race on it: order such calls.
//
// Returns 0 when the work was enqueued, a negative code otherwise.
int agb_rms_norm_bwd_noalloc(const void* grad, const void* x, const void* w, const float* rstd,
                             void* dx, float* dw, int64_t rows, int width, void* stream);

// Text of the last refusal or failure reported to this host thread ("" if none).
const char* agb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
