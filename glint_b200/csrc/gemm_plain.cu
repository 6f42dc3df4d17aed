// out[M, N] = A[M, K] * W[N, K]^T on the CUDA cores, 32-bit float accumulation.
//
// This is the matrix product of the true 32-bit path (tensor cores have no full-precision
// float mode) and the yardstick the tensor-core kernels are tested against.  Each output
// element is one fused-multiply-add chain over k = 0..K-1 in order, so a row's result does
// not depend on which other rows share the launch.  Weights are [out, in] row-major and are
// used untransposed, as the reference's matvec does (src/tensor/quantized.rs:1021-1044,
// src/transformer/forward.rs:546-557).
#include "common.cuh"

namespace glint {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename S>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const S* __restrict__ A, const S* __restrict__ W, float* __restrict__ out, int M,
                  int N, int K, float cap) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, k = idx & 15;
      const int gk = k0 + k;
      const int gm = m0 + row, gn = n0 + row;
      As[k][row] = (gm < M && gk < K) ? to_float(A[(size_t)gm * K + gk]) : 0.f;
      Ws[k][row] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * N + gn] = softcap(acc[i][j], cap);
    }
  }
}

}  // namespace glint

using namespace glint;

// cap > 0 applies cap * tanh(x / cap) to every output element.
GLINT_API int glint_gemm_plain(const void* A, const void* W, int dtype, float* out, int M, int N, int K,
                               float cap, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GLINT_OK;
  if (K <= 0) return GLINT_ERR_BAD_ARG;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  if (grid.y > 65535) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (dtype == GLINT_DTYPE_F32)
    gemm_plain_kernel<float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, out, M, N, K, cap);
  else if (dtype == GLINT_DTYPE_BF16)
    gemm_plain_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)A,
                                                               (const __nv_bfloat16*)W, out, M, N, K, cap);
  else
    return GLINT_ERR_BAD_ARG;
  return (int)cudaGetLastError();
}
