/* Layer-norm backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (which has no native code at all).  It exists for
 * code that runs where a device allocation is off the table: a plugin executing inside another runtime's
 * memory plan, a real-time inference loop that promised its host "no allocator calls after start-up", a
 * region that is being recorded for later replay, or a tool with a fixed memory budget.  Such callers cannot
 * use the package's normal layer-norm backward, because that one asks the framework allocator for a
 * temporary [ctas, hidden] buffer of partial parameter gradients on every call.
 *
 * Here that temporary lives in a fixed array inside the library image (8 MiB of device memory per GPU that
 * loads the library, held until the process exits).  The caller passes every input and every output; the
 * function itself calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *   dx, dgamma, dbeta = layer_norm_backward(dy, x, mean, rstd, gamma)
 *
 *   dy, x, dx : [rows, hidden] contiguous, bf16 (is_bf16 != 0) or fp16
 *   mean, rstd: [rows] fp32, as produced by the forward pass
 *   gamma     : [hidden] fp32
 *   dgamma, dbeta : [hidden] fp32, overwritten
 *
 * Limits: hidden must be a multiple of 8 and at most CW_NOALLOC_MAX_HIDDEN; rows >= 1.  Larger sizes are
 * rejected with CW_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *
 * First call on a device: looks up the device address of the built-in array (once per device, with that
 * device current).  Make that first call before any stream capture begins on the device.
 *
 * Sharing: every call on a device uses the same array, and the array keeps whatever the last call left in
 * it.  No word of it needs clearing, because each call writes every word it later reads.  Two calls that
 * may overlap on the GPU (different streams, no ordering between them) race on the array and give wrong
 * parameter gradients: order them on one stream or with events.
 *
 * Returns 0 on success, otherwise one of the codes below (nothing useful has been written in that case).
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CW_NOALLOC_MAX_HIDDEN 8192
#define CW_NOALLOC_MAX_CTAS 128

#define CW_NOALLOC_OK 0
#define CW_NOALLOC_ERR_TOO_LARGE 1  /* hidden > CW_NOALLOC_MAX_HIDDEN */
#define CW_NOALLOC_ERR_BAD_ARGUMENT 2 /* null pointer, rows < 1, hidden not a multiple of 8, misaligned tensor */
#define CW_NOALLOC_ERR_CUDA 3       /* symbol look-up or kernel launch failed; see cudaGetLastError().  The launches
                                      are checked with cudaPeekAtLastError(), so an error that the calling thread
                                      left pending from earlier work of its own is reported here as well */

int cw_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* mean, const float* rstd, const float* gamma,
                              void* dx, float* dgamma, float* dbeta, int rows, int hidden, int is_bf16,
                              cudaStream_t stream);

#ifdef __cplusplus
}
#endif
