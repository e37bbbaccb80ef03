// Row-wise arg-max that never allocates: its inter-CTA scratch is a fixed array inside the kernel
// library's own device image.  This entry point has no counterpart in the reference; it exists for
// callers that must not touch any allocator when they pick the next token.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest batch one call accepts (the scratch array holds this many rows and no more).
#define TELB_ARGMAX_STATIC_MAX_ROWS 256

// out[r] = index of the largest element of row r of `logits` (lowest index on ties).
//   logits   rows x vocab, row pitch `stride` elements, dtype 0 = fp16, 1 = bf16, 2 = fp32
//   out      rows x int32, device memory
// Returns 0, or -1 with the reason readable through telb_last_error().  rows above
// TELB_ARGMAX_STATIC_MAX_ROWS, vocab < 1 or an unknown dtype are refused, nothing is launched.
// `stream` (any stream, the default one included) and `logits` must belong to the device that is
// current in the calling thread: the scratch address is looked up for the current device, so a
// stream or a buffer of another device is refused with an error instead of being used.
//
// The first call on each device looks up the device address of the scratch array (with that device
// current), which may load the module; make that first call before any stream capture begins.
// All calls on one device share the one scratch array: each call clears it on `stream` before its
// kernel runs, so calls that overlap on different streams of a device race with one another and
// must be ordered by the caller.
int telb_argmax_static(const void* logits, int* out, int rows, int vocab, long long stride, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
