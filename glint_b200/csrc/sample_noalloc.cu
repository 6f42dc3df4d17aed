// Sampling without any allocation: the sampling kernel of sampling.cu, run on a scratch buffer
// that is part of the library's own device image.  See noalloc.h for who needs this and the rules.
// No counterpart in the reference.
#include "noalloc.h"

#include "common.cuh"

namespace glint {
// defined in sampling.cu
__global__ void sample_kernel(const float* src, long long src_stride, float* work, int V, const float* temperature,
                              const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                              int* out);
}  // namespace glint

// The scratch rows.  In host code this name is only a handle for cudaGetSymbolAddress: it is not a
// device pointer and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_rows[GLINT_NOALLOC_MAX_ROWS * GLINT_NOALLOC_MAX_VOCAB];

#define GLINT_NOALLOC_MAX_DEVICES 64
// Device address of g_noalloc_rows on each device, looked up on the first call there.
static float* g_noalloc_addr[GLINT_NOALLOC_MAX_DEVICES];

extern "C" __attribute__((visibility("default"))) int glint_sample_noalloc(
    const float* logits, long long row_stride, int rows, int vocab, const float* temperature, const int* top_k,
    const float* top_p, const float* min_p, const float* uniform, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !logits || !temperature || !top_k || !top_p || !min_p || !uniform || !out) return -1;
  if (rows > GLINT_NOALLOC_MAX_ROWS || vocab > GLINT_NOALLOC_MAX_VOCAB) return GLINT_NOALLOC_TOO_LARGE;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= GLINT_NOALLOC_MAX_DEVICES) return -1;
  float* scratch = g_noalloc_addr[device];
  if (!scratch) {
    // once per device, with that device current; two threads racing here store the same value
    e = cudaGetSymbolAddress((void**)&scratch, g_noalloc_rows);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_addr[device] = scratch;
  }
  // The kernel writes work[r, 0..vocab) from the logits before it reads any of it, so whatever an
  // earlier call left in the array is never seen.  Rows are packed with stride `vocab`.
  glint::sample_kernel<<<rows, 1024, 0, stream>>>(logits, row_stride, scratch, vocab, temperature, top_k, top_p,
                                                  min_p, uniform, out);
  return (int)cudaGetLastError();
}
