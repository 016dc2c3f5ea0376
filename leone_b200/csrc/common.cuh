// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Conventions used by every entry point in this directory:
//  * entry points are `extern "C"`, take raw device pointers, sizes and a
//    cudaStream_t, launch asynchronously and return a cudaError_t-compatible int
//    (0 = launched; negative = the sizes were refused, nothing was launched);
//  * `dtype` arguments: 0 = float32, 1 = bfloat16;
//  * kernels never trap: a bad index found on the device sets the status word
//    (atomicCAS on word 0 so the first fault wins) and the access is skipped.
//    The reference guards the same way
//    (crates/leone-cuda/cuda/ie_cuda.cu:2960-2966, 5610-5640).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace leone {

enum Status : int {
  kOk = 0,
  kBadTokenId = 1,      // detail: row, id
  kBadPage = 2,         // detail: token row, page id
  kBadPosition = 3,     // detail: token row, position
  kWaitTimeout = 4,     // detail: block, which wait
  kBadSequence = 5,     // detail: token row, sequence index
};

enum Refusal : int {
  kRefusedSize = -1,        // a size the kernel does not take
  kRefusedAlignment = -2,   // a pointer or stride that is not aligned as needed
  kRefusedDtype = -3,
};

__device__ __forceinline__ void set_status(int* status, int code, int d0, int d1, int d2 = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = d0;
    status[2] = d1;
    status[3] = d2;
  }
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// A value rounded to the storage type and back: what a later reader of T will see.
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_float<T>(from_float<T>(v));
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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

inline int launch_result() {
  return (int)cudaGetLastError();
}

// ---- thread-block clusters ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of every block of the cluster arrives and waits; shared-memory writes before the
// barrier are visible to the cluster's other blocks after it.  The hardware wait has no time
// limit, so it stands only where every thread is certain to arrive (after bounded loops).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Address of this block's shared-memory location `addr` in the block of rank `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_st_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void cluster_st_f32x2(uint32_t addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
// An arrival that publishes this thread's earlier reads and writes to the cluster, and the wait
// that makes the other blocks' published writes visible.
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// The two halves of a cluster barrier on their own: an arrival that orders nothing (it only says
// "this thread of this block is running"), and the wait that completes the phase.  Every thread
// pairs each arrival with one wait before it arrives again.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait;" ::: "memory");
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// ---- programmatic dependent launch -------------------------------------------------
// Kernels of a step are launched so that a kernel may start while its predecessor in the
// stream is still running.  A kernel calls pdl_trigger() early (its successor may then be
// scheduled once every block of this kernel has started) and pdl_wait() before it reads or
// writes anything a predecessor may still touch; pdl_wait() returns when the predecessor grid
// has completed and its writes are visible.  Work that depends on nothing written during the
// step (fetching weights) is done before pdl_wait().  Launched without the attribute, both
// calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// One switch per library image; off until the host turns it on.
inline int& pdl_flag() {
  static int enabled = 0;
  return enabled;
}

template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_flag() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return e == cudaSuccess ? launch_result() : (int)e;
}

// The same for a grid of thread-block clusters of shape `cluster`.
template <typename... KArgs, typename... Args>
inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = cluster.x;
  attrs[0].val.clusterDim.y = cluster.y;
  attrs[0].val.clusterDim.z = cluster.z;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = pdl_flag() ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return e == cudaSuccess ? launch_result() : (int)e;
}

}  // namespace leone
