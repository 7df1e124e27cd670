// Shared device helpers for the arle_b200 kernels (sm_100a).
//
// Conventions of every launcher in this directory:
//  * exported as extern "C", returns 0 on success, a cudaError_t (> 0) when the
//    launch failed, or a negative ARLE_E_* code when the sizes are refused;
//  * takes raw device pointers and the stream to launch on, allocates nothing;
//  * dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#define ARLE_E_UNSUPPORTED (-2)
#define ARLE_E_BADARG (-3)

#define ARLE_API extern "C" __attribute__((visibility("default")))

namespace arle {

constexpr int kWarp = 32;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
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

// Block-wide sum for blocks of up to 1024 threads; every thread gets the result.
// `scratch` must hold 33 floats of shared memory.  The order of the additions is
// fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
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
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch.  Every kernel of this library starts with
// pdl_launch_dependents() (the next kernel of the stream may be scheduled as soon as
// all CTAs of this one have started) and calls pdl_wait() before it first touches
// memory that an earlier kernel may have written (until then it may only set up
// barriers and fetch weights, which no kernel writes).  Both are no-ops for a kernel
// launched in the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Bit 0: every kernel is launched with programmatic stream serialisation allowed; bit 1:
// the weight-streaming products only (they fill their weight ring while the kernel before
// them finishes).  Off by default.
inline int& pdl_enabled() {
  static int on = 0;
  return on;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic-launch attribute
// (and a cluster dimension when cluster > 1).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_as(bool programmatic, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, int cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (programmatic) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 int cluster, Args&&... args) {
  return launch_kernel_as((pdl_enabled() & 1) != 0, kernel, grid, block, smem, stream, cluster, std::forward<Args>(args)...);
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace arle
