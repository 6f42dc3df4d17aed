// Shared device helpers of the glint_b200 kernels (sm_100a).
//
// Storage types are float or __nv_bfloat16; arithmetic is 32-bit float everywhere.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GLINT_OK 0
// Negative codes are refusals made on the host before any launch; positive codes are cudaError_t.
#define GLINT_ERR_BAD_ARG (-1)
#define GLINT_ERR_UNSUPPORTED_SIZE (-2)
#define GLINT_ERR_DEVICE_TIMEOUT (-3)

#define GLINT_DTYPE_F32 0
#define GLINT_DTYPE_BF16 1

#define GLINT_API extern "C" __attribute__((visibility("default")))

namespace glint {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float softcap(float x, float cap) {
  // cap * tanh(x / cap); cap <= 0 means no cap
  return cap > 0.f ? cap * tanhf(x / cap) : x;
}

__device__ __forceinline__ float gelu_tanh(float v) {
  return 0.5f * v * (1.0f + tanhf(0.7978846f * (v + 0.044715f * v * v * v)));
}

}  // namespace glint
