/* glint_sample_noalloc: token sampling for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in HamadAndrabi/glint; it exists for hosts of this
 * library that cannot call cudaMalloc themselves and cannot let a library do it for them:
 * control loops that fixed their whole device-memory budget at start-up and treat any later
 * allocation as a fault; processes that share a GPU under a hard memory quota, where an
 * allocation in mid-run may simply fail; and programs whose device memory is entirely owned by
 * another component's pool, so that nothing is left for the driver's allocator to hand out.
 *
 * The regular sampler (glint_sample) is given its scratch row-buffer by the caller.  This variant
 * owns one: a fixed array inside the library's device image, GLINT_NOALLOC_MAX_ROWS rows of
 * GLINT_NOALLOC_MAX_VOCAB floats (8 MiB).  Every GPU that loads the library holds that array until
 * the process exits, whether or not this function is ever called.
 *
 * Rules for callers:
 *  - rows <= GLINT_NOALLOC_MAX_ROWS and vocab <= GLINT_NOALLOC_MAX_VOCAB, else the call returns
 *    GLINT_NOALLOC_TOO_LARGE and launches nothing.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *    no allocation).  Make that first call outside any stream capture; later calls only launch.
 *  - All calls share the one array.  Each call overwrites the part it uses before reading it, so
 *    nothing needs clearing between calls; but two calls whose kernels overlap on the GPU (different
 *    streams, or graphs replayed concurrently) race on it.  Serialize them on one stream.
 *  - Inputs and outputs are the caller's device memory, exactly as for glint_sample.
 */
#ifndef GLINT_NOALLOC_H
#define GLINT_NOALLOC_H

#include <cuda_runtime.h>

#define GLINT_NOALLOC_MAX_ROWS 8
#define GLINT_NOALLOC_MAX_VOCAB 262144
#define GLINT_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C" {
#endif

/* logits: rows x vocab floats, row stride `row_stride` elements.  Per row: temperature (> 0),
 * top_k (0 = off), top_p (1 = off), min_p (0 = off), one uniform draw in [0, 1).  out: rows ints.
 * Returns 0, GLINT_NOALLOC_TOO_LARGE, -1 for a bad argument, or a positive cudaError_t. */
int glint_sample_noalloc(const float* logits, long long row_stride, int rows, int vocab,
                         const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                         const float* uniform, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
