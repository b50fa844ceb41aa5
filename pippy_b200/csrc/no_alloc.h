// Allocation-free entry point of libpippy_b200.so.  It has no counterpart in the reference.
//
// Who needs it: callers that are not allowed to allocate device memory at the point of the call, for example code
// running inside a region where the allocator is frozen, a plugin loaded into a process whose memory budget is
// fixed up front, or a host that drives the library through this C ABI without PyTorch and has no workspace to
// hand over.  The regular entry point (pb_norm_bwd) needs a scratch buffer from its caller; this one brings its own.
//
// pb_rmsnorm_bwd_noalloc computes the RMSNorm backward:
//     dx[T, H] (bf16)      gradient of the input
//     dw_f32[H] (fp32)     gradient of the weight; written, or added to when `accumulate` is non-zero
// from dy[T, H], x[T, H], w[H] (bf16) and rstd[T] (fp32, as produced by pb_norm_fwd).  H must be a multiple of 8.
//
// Scratch: a file-scope device array of 128 x 2 x 8192 floats (8 MiB) that every GPU loading the library holds until
// the process exits.  H above pb_rmsnorm_bwd_noalloc_max_hidden() (8192) is rejected with -2; nothing is
// truncated.  The call makes no cudaMalloc/cudaFree and calls no allocating library routine.
//
// Work split: the rows are spread over at most 128 CTAs (the number of partial rows the array holds), whatever T is;
// the regular entry point uses two CTAs per SM.  dx is the same bit for bit, dw differs from the regular entry
// point's by the order in which the per-CTA partial sums are added (fp32 rounding only).
//
// First call on each device: the entry point resolves the array's device address (cudaGetSymbolAddress) with that
// device current, and caches it (under a mutex, so concurrent first calls from several host threads are safe).
// Make that first call outside any stream capture.
//
// Sharing: all calls on a device use the same array and it keeps the previous call's contents.  Every partial row is
// fully rewritten before it is read, so nothing has to be cleared, but two calls that overlap on the GPU (different
// streams) race on it: serialise them.
//
// Returns 0 on success, a negative value for a rejected argument, a positive cudaError_t otherwise.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int pb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_f32,
                           int accumulate, int T, int H, void* stream);
int pb_rmsnorm_bwd_noalloc_max_hidden(void);

#ifdef __cplusplus
}
#endif
