// Shared host and device helpers: checked launches, dtype-generic loads and stores, reductions.
//
// Host side: every entry point checks sizes and pointers with FTK_REQUIRE before it launches and
// reads the launch status afterwards; the text of the first failure is kept per thread for
// ftk_last_error().  (The reference wraps its launches the same way: TensorMatcher / RuntimeCheck /
// LaunchKernel in python/freetoken/kernel/csrc/include/freetoken/{tensor.h,utils.h,utils.cuh}.)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "api.h"

namespace ftk {

void set_error(const char* fmt, ...);
// Counts a launch under the name of the kernel form it took (`name` must be a string literal);
// ftk_variant_counts() reports the counts.
void note_variant(const char* name);

#define FTK_REQUIRE(cond, ...)        \
  do {                                \
    if (!(cond)) {                    \
      ftk::set_error(__VA_ARGS__);    \
      return 1;                       \
    }                                 \
  } while (0)

#define FTK_LAUNCH_CHECK(name)                                              \
  do {                                                                      \
    cudaError_t e_ = cudaGetLastError();                                    \
    if (e_ != cudaSuccess) {                                                \
      ftk::set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
      return 2;                                                             \
    }                                                                       \
  } while (0)

// Every kernel is launched so that it may start while the kernel before it in the stream is still
// running (programmatic dependent launch): a kernel calls pdl_wait() before it touches anything that
// an earlier kernel wrote or still reads, and pdl_trigger() when the next kernel's blocks may come
// onto the SMs.  A kernel that never triggers lets the next one in when it ends.  FTK_PDL=0 in the
// environment launches everything the plain way.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// The same for a kernel whose CTAs come in clusters of `cluster` consecutive blocks.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_clusters(void (*kernel)(KArgs...), int cluster, dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#define FTK_LAUNCH(kernel, grid, block, smem, stream, ...) \
  ftk::launch_kernel(kernel, dim3(grid), dim3(block), (size_t)(smem), (cudaStream_t)(stream), __VA_ARGS__)

inline bool dtype_ok(int d) { return d == FTK_F32 || d == FTK_BF16; }
inline int dtype_size(int d) { return d == FTK_F32 ? 4 : 2; }

// ---------------------------------------------------------------- device helpers
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over the block in a fixed order (warp shuffles, then warp 0 over the warp sums); every
// thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Gated activations on float inputs (python/freetoken/kernel/triton/activation.py:96-107).
__device__ __forceinline__ float gated_act(float g, float u, int act, float alpha, float limit) {
  if (act == FTK_ACT_SILU) return g / (1.f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

// The same with the fast exponential and division (about 2^-21 relative each): for results that are rounded
// to bfloat16 right away.
__device__ __forceinline__ float gated_act_fast(float g, float u, int act, float alpha, float limit) {
  if (act == FTK_ACT_SILU) return __fdividef(g, 1.f + __expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return __fdividef(g, 1.f + __expf(-alpha * g)) * (u + 1.f);
}

}  // namespace ftk
