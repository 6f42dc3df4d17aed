// Shared device helpers of the glint_b200 kernels (sm_100a).
//
// Storage types are float or __nv_bfloat16; arithmetic is 32-bit float everywhere.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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


// ---- thread-block cluster -----------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of this block's shared address `addr` in block `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float cluster_load(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched with launch_kernel() may begin while its predecessor on the stream is still
// finishing: everything up to pdl_wait() (set-up, loads of weights, which no kernel writes)
// overlaps the predecessor's tail; pdl_wait() returns once the predecessor has completed and its
// writes are visible.  pdl_launch_dependents() lets the successor begin in the same way.  Under
// an ordinary launch both are no-ops.  GLINT_PDL=0 in the environment switches the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// What every kernel here does: wait for the predecessor and only then let the successor start, so
// that at most one kernel starts under another.  A kernel that released its successor before its
// own wait let a whole chain of kernels start under one that was still streaming: measured on a
// decode step with 36,864-feature products, the idle blocks of the kernels two and three places
// behind took the SMs' registers from the blocks that still had weights to stream, and the step
// took half as long again (1.79 -> 1.21 ms for four such layers and the output head).
__device__ __forceinline__ void pdl_wait_release() {
  pdl_wait();
  pdl_launch_dependents();
}
static inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("GLINT_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// `cluster_z` > 1 launches the grid as thread-block clusters of that many blocks along z.  Such a
// launch does not start early under its predecessor: measured, clusters placed among the blocks
// of a kernel that is still running cost a decode step 10 us per layer.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                                cudaStream_t stream, int cluster_z, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = (pdl_enabled() && cluster_z <= 1) ? 1 : 0;
  cfg.numAttrs = 1;
  if (cluster_z > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = (unsigned)cluster_z;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args... args) {
  return launch_kernel_cluster(kernel, grid, block, smem, stream, 1, args...);
}

}  // namespace glint
