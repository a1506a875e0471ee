// Shared device helpers and the launch wrapper used by every kernel in this library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rlz {

// ---- launch bookkeeping (defined in runtime.cu) ------------------------------------------
void note_launch();
bool pdl_enabled();

// Launch `kernel` on `stream`.  When programmatic dependent launch is enabled the kernel may
// start while its predecessor drains; every kernel therefore calls pdl_wait() before touching
// data produced by earlier kernels.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
  }
  note_launch();
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Same, with a thread-block cluster shape (1,1,1 = no cluster attribute).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x; attr[n].val.clusterDim.y = cluster.y; attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  cfg.attrs = n ? attr : nullptr; cfg.numAttrs = n;
  note_launch();
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Dynamic shared memory above the default limit has to be opted into per kernel AND per device (the attribute belongs to
// the function on one device).  One instance per kernel instantiation remembers what each device has been set to; a
// repeated call from another thread at worst sets the same attribute twice.
struct SmemOptIn {
  size_t bytes[64] = {};
  template <typename K>
  cudaError_t ensure(K kernel, size_t smem, size_t default_limit = 48 * 1024) {
    if (smem <= default_limit) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int slot = dev & 63;
    if (smem <= bytes[slot]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) bytes[slot] = smem;
    return e;
  }
};

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// 8-byte {payload, epoch} pairs exchanged between GPUs: one store / load each, never torn
__device__ __forceinline__ void st_pair_sys(uint2* p, uint32_t a, uint32_t b) {       // one 8-byte store, visible system-wide
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
  uint2 v; asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory"); return v;
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
// Block-wide sum; `red` is >= 33 floats of shared memory.  All threads must call.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -3.4e38f;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
#endif

// activation / combine codes shared with the Python side
enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2 };
enum { COMBINE_ADD = 0, COMBINE_SILU_MUL = 1, COMBINE_GELU_MUL = 2 };
enum { NORM_NONE = 0, NORM_RMS = 1, NORM_LAYER = 2 };

}  // namespace rlz
