// SPDX-License-Identifier: Apache-2.0
/* RMSNorm backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for users of this library.
 *
 * Who needs it: code that runs where a device allocation is off limits.  Typical cases are a host process that
 * has handed the whole GPU to one memory pool and forbids anything outside it, a latency-critical loop in which
 * the implicit device synchronisation of cudaMalloc/cudaFree would stall every stream, and plain C or C++ hosts
 * that link this library without the tensor framework and therefore have no caching allocator to lean on.
 * The tensor-based operator (`torch.ops.atb200.rmsnorm_bwd`) allocates its output and a block of partial sums on
 * every call; this function allocates nothing, ever.
 *
 * What it computes (same math as the tensor-based operator):
 *     dx[t, :] = rstd[t] * (dy[t, :] * w - x[t, :] * rstd[t]^2 * mean(dy[t, :] * w * x[t, :]))
 *     dw[:]    = sum_t dy[t, :] * x[t, :] * rstd[t]
 * dy, x, dx are bf16 [rows, hidden] (row-major, 16-byte aligned), w is bf16 [hidden], rstd is fp32 [rows] as
 * produced by the forward pass, dw is fp32 [hidden].  All pointers are device pointers owned by the caller and
 * must belong to the device that is current at the call (the scratch array that is used is that device's); the
 * function looks each one up in the driver's address map and refuses host memory or another GPU's memory.
 *
 * Scratch: the per-block partial sums of dw live in a fixed array inside the library image
 * (148 x 8192 floats = 4.6 MiB), which every GPU that loads the library holds until the process exits.
 * Limit: hidden must be a multiple of 8 and at most ATB_NOALLOC_MAX_HIDDEN; larger sizes are refused.
 *
 * Sharing: all calls on one device use the same scratch array.  The part a call uses is fully overwritten before
 * it is read, so nothing has to be cleared between calls, but two calls that overlap on the GPU (different
 * streams, or different host threads launching at the same time) race on it.  Serialise them on one stream.
 *
 * First call on a device: it looks up the device address of the scratch array (one runtime query, no
 * allocation) and remembers it.  Make that first call with the intended device current, and before starting any
 * stream capture on that device.
 *
 * Returns 0 on success.  On failure returns a non-zero code and, when `err` is not NULL, writes a
 * NUL-terminated message of at most `err_len` bytes:  1 = bad argument (null pointer, misalignment, size beyond
 * the limit, memory that is not the current device's), 2 = the CUDA runtime reported an error (message carries
 * its text).
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ATB_NOALLOC_MAX_HIDDEN 8192
#define ATB_NOALLOC_MAX_BLOCKS 148

int atb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                            long long rows, int hidden, void* cuda_stream, char* err, unsigned long err_len);

#ifdef __cplusplus
}
#endif
