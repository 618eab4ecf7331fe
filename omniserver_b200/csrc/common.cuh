// Shared helpers for the sm_100a kernels: storage types, conversions, warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#define OSB_API extern "C" __attribute__((visibility("default")))

// dtype codes used across the C interface
enum OsbDtype : int { OSB_F32 = 0, OSB_BF16 = 1 };

// error codes returned by the launch functions (besides cudaError values, which are < 10000)
enum OsbStatus : int {
  OSB_OK = 0,
  OSB_ERR_BAD_DTYPE = 10001,
  OSB_ERR_BAD_SHAPE = 10002,
  OSB_ERR_UNSUPPORTED = 10003,
  OSB_ERR_TOO_LARGE = 10004,
};

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result. The order of the
// additions depends only on blockDim, so a row's result does not depend on what else is in the grid.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect smem32 from a previous use
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem32[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem32[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

static inline int osb_last_error() { return (int)cudaGetLastError(); }

// Programmatic dependent launch: a kernel launched through osb_launch may start while the kernel
// before it in the stream is finishing; it must call pdl_wait() before it reads or writes anything
// the earlier kernel touches (until then only its own set-up runs), and calls pdl_trigger() when the
// kernel after it may begin to launch. Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int& osb_pdl_enabled() {
  static int v = 1;
  return v;
}

// cluster_x > 1 launches thread-block clusters of that many CTAs along x (gridDim.x must be a multiple).
template <typename... KArgs, typename... Args>
static inline int osb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (osb_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
static inline int osb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  return osb_launch_cluster(kernel, grid, block, smem, stream, 1, std::forward<Args>(args)...);
}

// Dispatch over the two storage types: f(Tag<T>{}) is called with T = float or bf16.
template <typename T> struct Tag { typedef T type; };

template <typename F> static inline int osb_dispatch(int code, F&& f) {
  if (code == OSB_F32) return f(Tag<float>{});
  if (code == OSB_BF16) return f(Tag<bf16>{});
  return OSB_ERR_BAD_DTYPE;
}
#define OSB_T(tag) typename decltype(tag)::type
