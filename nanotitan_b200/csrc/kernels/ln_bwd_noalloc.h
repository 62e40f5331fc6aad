// LayerNorm backward for callers that must not allocate.
//
// This entry point has no counterpart in the reference.  It exists for callers that cannot
// call cudaMalloc (or any allocating routine) at the point where they need the kernel: code
// running while a CUDA graph is being captured, callers living inside another framework's
// memory pool with no allocator handle of their own, real-time loops that may not take the
// allocator lock, and plain C programs that link this library without PyTorch.  The regular
// entry point (`layer_norm_bwd` of the Python module) asks PyTorch's allocator for its outputs
// and for a block of partial sums; this one takes every output from the caller and keeps its
// partial sums in a fixed array that is part of the library image.
//
// Limits and rules:
//   * d (row width) <= NT_LN_NOALLOC_MAX_D; larger rows are rejected with NT_LN_NOALLOC_TOO_LARGE.
//     Any number of rows is accepted.
//   * The scratch array (NT_LN_NOALLOC_SCRATCH_BYTES, 8 MiB) is resident on every GPU that loads
//     the library, until the process exits.
//   * The first call on a device looks up the device address of the scratch array
//     (cudaGetSymbolAddress).  Make that first call outside any stream capture, with the device
//     that owns the buffers current.  Several host threads may make their first calls at the same
//     time (the per-device address cache is atomic); the cache is keyed by device ordinal and
//     assumes the device is not reset (cudaDeviceReset) while the library stays loaded.
//   * All calls share the one scratch array, and it keeps what the previous call left in it; the
//     kernel clears the part it uses.  Two calls whose kernels overlap on the GPU (different
//     streams, no dependency between them) race on it: order them.
//   * Nothing is allocated or freed, by CUDA or by any library, on any call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NT_LN_NOALLOC_MAX_D 4096
#define NT_LN_NOALLOC_ROWS_OF_PARTIALS 256
#define NT_LN_NOALLOC_SCRATCH_BYTES (2 * NT_LN_NOALLOC_ROWS_OF_PARTIALS * NT_LN_NOALLOC_MAX_D * 4)

#define NT_LN_NOALLOC_OK 0
#define NT_LN_NOALLOC_BAD_ARGUMENT (-1)  /* null pointer, rows < 0, d < 1, unknown dtype */
#define NT_LN_NOALLOC_TOO_LARGE (-2)     /* d > NT_LN_NOALLOC_MAX_D */
#define NT_LN_NOALLOC_CUDA_ERROR (-3)    /* a CUDA call failed; the message names it */

// dx[rows, d] (same dtype as x), dgamma[d], dbeta[d] (fp32) from dy, x, gamma and the forward's
// per-row mean / rstd (fp32).  dtype: 0 = fp32, 1 = fp16, 2 = bf16 for dy, x, gamma, dx.
// `stream` is a cudaStream_t (null = default stream).  On failure a description is copied into
// `err` (when err != null and err_len > 0) and a negative code is returned.
int nt_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                              void* dx, float* dgamma, float* dbeta, long long rows, int d, int dtype, void* stream,
                              char* err, int err_len);

#ifdef __cplusplus
}
#endif
