// An allocation-free entry point.  It has NO counterpart in the reference (which has no native code at all); it exists
// for users of this library whose code is not allowed to allocate device memory.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward (same math as fth_rmsnorm_bwd in api.h):
//     dx = rstd * (g*w - xhat * mean(g*w*xhat)) + dres,   dw_main_grad += sum over rows of g * xhat,
// with g = dy * out_scale and xhat = x * rstd.  dy / x / dres / dx are bf16 [M, H], w is bf16 [H], rstd fp32 [M],
// dw_main_grad fp32 [H] (accumulated into).  dres may be NULL.
//
// Who this is for: callers that cannot call cudaMalloc where they run the op — a host runtime whose device memory is
// one fixed arena planned ahead of time, a plug-in running inside somebody else's process that must not touch the
// allocator, a real-time or safety-certified loop where allocation is forbidden after start-up, or code that would
// otherwise have to size and thread a scratch buffer through layers that do not own any memory.  fth_rmsnorm_bwd needs
// such a buffer (fth_rmsnorm_bwd_blocks(M, H) x H floats of per-block partial weight-gradient sums); this variant keeps
// it inside the library instead.
//
// What it does NOT do: it never calls cudaMalloc, cudaFree or any allocating library routine.  Its scratch is a
// file-scope device array of 296 x 4096 floats (4.625 MiB) that every GPU loading this library holds until the process
// exits.
//
// Limits: H <= 4096 and H % 8 == 0 (larger or odd H returns a negative code and writes a message into `err`); any M.
// Device ordinals below 64.
//
// First call on a device: the library looks up the device address of its scratch array (cudaGetSymbolAddress) with the
// caller's current device.  That is a one-time set-up step; make the first call on each device outside of any CUDA
// stream capture.  Later calls only launch kernels on `stream`.
//
// Sharing: all calls on a device use the same scratch array and the array keeps whatever the last call left in it.  The
// kernels overwrite every element they later read, so no clearing is needed between calls; but two calls that can run at
// the same time on one GPU (different streams without an ordering between them, or two host threads) race on it.  Order
// them on one stream or with events.  (The one-time address look-up itself may be done by two host threads at once on
// their first calls: both store the same value into the per-device slot, an unsynchronised but idempotent write.)
//
// Returns 0 on success; on failure a negative code, and if `err` is not NULL a zero-terminated message of at most
// `err_len` bytes.
int fth_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                            float* dw_main_grad, int M, int H, float out_scale, cudaStream_t stream, char* err,
                            size_t err_len);

#ifdef __cplusplus
}
#endif
