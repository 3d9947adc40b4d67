// Shared helpers of the sm_100a kernels: dtype codes, loads that widen to
// float32, stores that round to the output type, and block reductions whose
// summation order is fixed (so a result never depends on launch geometry).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LRM_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python wrappers
enum : int { LRM_F32 = 0, LRM_BF16 = 1 };

// error codes returned by host entry points (0 = ok, >0 = cudaError_t)
enum : int { LRM_BAD_ARGUMENT = -1, LRM_UNSUPPORTED = -2, LRM_DEVICE_STATUS = -3 };

#define LRM_LAUNCH_CHECK()                              \
  do {                                                  \
    cudaError_t e__ = cudaGetLastError();               \
    if (e__ != cudaSuccess) return static_cast<int>(e__); \
  } while (0)

// --- programmatic dependent launch ------------------------------------------------------
// Kernels of a step run back to back on one stream. With the launch attribute below a kernel
// may be scheduled while its predecessor still runs; it then does whatever does not depend on
// the predecessor (index arithmetic, prefetching weights) and calls pdl_wait() before it
// reads or writes anything the predecessor touches. pdl_wait() returns once the predecessor
// grid has completed and its writes are visible. pdl_trigger() lets the successor be
// scheduled as soon as every CTA of this grid has called it (or exited).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_lrm_pdl;  // 1: launch with programmatic stream serialization (set by lrm_set_pdl)

template <typename... KArgs, typename... Args>
inline cudaError_t lrm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = g_lrm_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

#define LRM_LAUNCH(kernel, grid, block, smem, stream, ...)                                  \
  do {                                                                                      \
    cudaError_t e__ = lrm_launch(kernel, grid, block, smem, stream, __VA_ARGS__);           \
    if (e__ != cudaSuccess) return static_cast<int>(e__);                                   \
  } while (0)

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

// Sum over a block of up to 1024 threads; every thread gets the same value.
// Order: butterfly inside each warp, then warp totals added in warp order.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < warps; ++w) total += scratch[w];
  return total;
}
