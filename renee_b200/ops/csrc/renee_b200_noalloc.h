/* Allocation-free entry point of the renee_b200 kernel library.
 *
 * This function has no counterpart in the reference implementation.  It exists for callers that
 * are not allowed to allocate device memory at the point where they need a kernel: code running
 * inside a memory pool that has been frozen for the rest of the job, plugins loaded into a host
 * application that owns every byte of the GPU, and real-time loops in which cudaMalloc (which
 * may synchronise the whole device) must never happen.  Such callers can still pass their own
 * input and output buffers, but they cannot provide the scratch memory that the regular entry
 * point rb_colsum expects, so here the scratch is part of the library image.
 *
 *   int rb_colsum_noalloc(int dtype, const void* x, void* out, int rows, int N, cudaStream_t st);
 *
 *   out[c] = sum over r of x[r, c]   for a row-major [rows, N] matrix, accumulated in fp32.
 *   dtype: 0 = float, 1 = bfloat16, 2 = half (x and out have the same type).
 *   N must be a multiple of 8 and at most rb_colsum_noalloc_max_cols() (8192); larger inputs are
 *   refused with return code -10 and a message on stderr.  Other non-zero codes: -1 unknown dtype
 *   code and -3 bad shape (both returned before anything is queued on the stream), -11/-12/-13 CUDA
 *   runtime failure during set-up, a positive value is a cudaError_t of the launch.
 *
 * Things to know:
 *   - The scratch is a static device array of 8 * 8192 floats (256 KB) plus a 256-byte counter block.
 *     Every GPU that loads the library holds them until the process exits.
 *   - The function calls no cudaMalloc, cudaFree or allocating library routine.
 *   - The first call on each device looks up the device addresses of the scratch symbols.  Make
 *     that first call with the device current and before any stream capture is begun.
 *   - All calls on a device share the same scratch.  Each call clears what it needs at its start
 *     (stream-ordered), so back-to-back calls on one stream are fine, but two calls whose kernels
 *     can overlap on the GPU (different streams without an ordering between them) race on the
 *     scratch and give wrong sums.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int rb_colsum_noalloc(int dtype, const void* x, void* out, int rows, int N, cudaStream_t st);
int rb_colsum_noalloc_max_cols(void);

#ifdef __cplusplus
}
#endif
