// Shared device helpers of the sm_100a kernels: element conversion, warp and
// block reductions, and the error word that kernels set instead of trapping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <utility>

namespace tk {

// Element types of activations, weights and cache pages, as passed over the C ABI.
enum DType : int { kF32 = 0, kBF16 = 1 };

// Error codes written to the 4-int error word (code, detail0, detail1, detail2).
enum ErrCode : int {
  kErrNone = 0,
  kErrTokenId = 1,    // token id outside [0, vocab)
  kErrPage = 2,       // page id outside the pool, or page index outside the table row
  kErrPosition = 3,   // negative position
  kErrRequest = 4,    // request row outside the batch
  kErrWait = 5,       // a bounded wait on a barrier ran out
};

__device__ __forceinline__ void set_error(int* err, int code, int d0, int d1, int d2) {
  if (err == nullptr) return;
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = d0;
    err[2] = d1;
    err[3] = d2;
  }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

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

// Sum over a thread block; `scratch` holds at least 32 floats of shared memory.
// Every thread receives the result.  Safe to call repeatedly with the same scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// Programmatic dependent launch.  Every kernel of this library is launched so that it may
// start while the kernel before it in the stream is still running, lets the kernel after it
// start early in turn (pdl_trigger at its top), and calls pdl_wait before it touches anything
// that an earlier kernel wrote and before it writes anything itself.  What runs before
// pdl_wait (index arithmetic, barrier set-up, loads of weights, which no kernel writes)
// overlaps the tail of the previous kernel.  Without the launch attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// TOKAMAK_B200_PDL=0 in the environment switches the launch attribute off.
inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("TOKAMAK_B200_PDL");
    enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Thread-block clusters: rank, barrier over all threads of the cluster, and reads of another
// block's shared memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// Sum over the blocks 0 .. csize-1 (at most 8) of a cluster of the four floats at the same
// shared-memory address of each, added in the order of the ranks.  All loads are requested before
// the first sum, so that their latencies over the cluster's network overlap.
__device__ __forceinline__ float4 cluster_sum_f32x4(uint32_t local_smem_addr, int csize) {
  float4 v[8];
#pragma unroll
  for (int rk = 0; rk < 8; ++rk) {
    if (rk < csize) v[rk] = ld_cluster_f32x4(local_smem_addr, (uint32_t)rk);
  }
  float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
  for (int rk = 0; rk < 8; ++rk) {
    if (rk < csize) { sum.x += v[rk].x; sum.y += v[rk].y; sum.z += v[rk].z; sum.w += v[rk].w; }
  }
  return sum;
}


// The same with thread-block clusters of the given shape.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Clusters of the blocks of every grid.z column.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster_z(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, unsigned cluster_z, Args&&... args) {
  return launch_cluster(kernel, grid, block, smem, stream, dim3(1, 1, cluster_z), std::forward<Args>(args)...);
}

}  // namespace tk

// Dispatch a templated launch on the element type code.
#define TK_DISPATCH_DTYPE(code, T, ...)                 \
  do {                                                  \
    if ((code) == tk::kF32) {                           \
      using T = float;                                  \
      __VA_ARGS__;                                      \
    } else if ((code) == tk::kBF16) {                   \
      using T = __nv_bfloat16;                          \
      __VA_ARGS__;                                      \
    } else {                                            \
      return (int)cudaErrorInvalidValue;                \
    }                                                   \
  } while (0)

#define TK_API extern "C" __attribute__((visibility("default")))
