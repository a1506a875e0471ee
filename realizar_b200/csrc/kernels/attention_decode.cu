// Flash-decode GQA attention over a paged bf16 KV cache, one new token per sequence, with the
// work that surrounds it in a decode layer fused in:
//   * per-head RMSNorm of q/k (QK-norm models), RoPE (NORM / NEOX, partial rotary) on q and k
//   * append of the new k/v row to the paged cache
//   * split-K over the context (grid.y) merged without a second launch.  Up to 8 splits the CTAs
//     of one (sequence, kv-head group) form a thread-block cluster and CTA 0 merges the others'
//     partial results straight out of their shared memory (DSMEM); beyond 8 splits the partials go
//     through global memory and the last CTA to finish (atomic ticket) merges them; one split
//     writes its result directly.
//   * optional sliding window (attend to the last `window` positions only) and a precomputed
//     cos/sin table for RoPE (no transcendental math on the critical path).
//
// Cache layout: k_cache / v_cache = bf16 [num_pages, n_kv_heads, PAGE, head_dim]; a
// sequence's pages are listed in page_table[b, :].  Positions are read from device memory so
// the launch is replayable inside a CUDA graph; positions[b] < 0 marks an empty batch slot.
//
// Replaces the reference's rope*/kv_cache_scatter*/incremental_attention*/multi_warp_attention*/
// flash_decoding_chunk+reduce kernels (src/cuda/executor/kv_scatter.rs:15-388,
// src/cuda/executor/flash_decoding_graphed.rs:14-209, src/cuda/executor/batch.rs:18-400).
#include "common.cuh"
#include <stdlib.h>
#include "attn_decode_static.h"
#include "attention_decode_body.cuh"
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <math.h>

namespace rlz {

template <int GT, int MERGE, int DEEP, int Q8>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __grid_constant__ AttnDecodeParams p) {
  __shared__ AttnSmem<GT, MERGE> sm;
  extern __shared__ __align__(128) uint8_t att_ring[];      // streamed mode (DEEP == 2): the K/V page ring
  pdl_launch_dependents();
  pdl_wait();
  attn_decode_body<GT, MERGE, DEEP, Q8, 0, false>(p, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)threadIdx.x, sm, 0, att_ring);
}

// tensor-core mode: head_dim is a template parameter
template <int GT, int MERGE, int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_mma_kernel(const __grid_constant__ AttnDecodeParams p) {
  __shared__ AttnSmem<GT, MERGE> sm;
  extern __shared__ __align__(128) uint8_t att_ring[];
  pdl_launch_dependents();                                  // the body waits for the preceding kernel itself, after its K/V prefetch
  attn_decode_body<GT, MERGE, 3, 0, 0, false, HD, true>(p, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)threadIdx.x, sm, 0, att_ring);
}

template <int GT, int MERGE, int HD>
static cudaError_t launch_attn_mma(const AttnDecodeParams& p, dim3 grid, dim3 block, dim3 cl, cudaStream_t st) {
  const size_t ring = (size_t)ATT_RING * 64 * (HD == 80 ? 2 * HD : 2 * HD + 16);       // row bytes as in the kernel
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(attn_decode_mma_kernel<GT, MERGE, HD>, ring, 0); e != cudaSuccess) return e;   // static shared memory comes on top: always opt in
  return launch_cluster(attn_decode_mma_kernel<GT, MERGE, HD>, grid, block, cl, ring, st, p);
}
template <int GT, int MERGE>
static cudaError_t launch_attn_mma_hd(const AttnDecodeParams& p, dim3 grid, dim3 block, dim3 cl, cudaStream_t st) {
  switch (p.head_dim) {
    case 64: return launch_attn_mma<GT, MERGE, 64>(p, grid, block, cl, st);
    case 80: return launch_attn_mma<GT, MERGE, 80>(p, grid, block, cl, st);
    case 96: return launch_attn_mma<GT, MERGE, 96>(p, grid, block, cl, st);
    default: return launch_attn_mma<GT, MERGE, 128>(p, grid, block, cl, st);
  }
}
template <int GT>
static cudaError_t launch_attn_mma_merge(const AttnDecodeParams& p, int merge, dim3 grid, dim3 block, dim3 cl, cudaStream_t st) {
  return merge == MERGE_NONE ? launch_attn_mma_hd<GT, MERGE_NONE>(p, grid, block, cl, st) : launch_attn_mma_hd<GT, MERGE_CLUSTER>(p, grid, block, cl, st);
}

// launch one instantiation; `ring` bytes of dynamic shared memory (0 unless streamed)
template <int GT, int MERGE, int DEEP, int Q8>
static cudaError_t launch_attn(const AttnDecodeParams& p, dim3 grid, dim3 block, dim3 cl, size_t ring, cudaStream_t st) {
  static SmemOptIn opt;                                       // above the default limit once the static part is added: opt in
  if (cudaError_t e = opt.ensure(attn_decode_kernel<GT, MERGE, DEEP, Q8>, ring, 16 * 1024); e != cudaSuccess) return e;
  return launch_cluster(attn_decode_kernel<GT, MERGE, DEEP, Q8>, grid, block, cl, ring, st, p);
}

}  // namespace rlz

namespace rlz {

// Validate and launch: picks the head-group tile, the K/V access mode and the merge strategy.
static int attn_decode_dispatch(const AttnDecodeParams& p, cudaStream_t st) {
  if (p.head_dim % 8 || p.head_dim > 128 || p.head_dim < 8) return -1;
  if (p.n_kv_heads < 1 || p.n_heads % p.n_kv_heads || p.splits < 1 || p.batch < 1) return -2;
  if (p.rope_dim > p.head_dim || (p.rope_dim & 1)) return -3;
  if (((uintptr_t)p.k_cache & 15) || ((uintptr_t)p.v_cache & 15)) return -4;
  if (p.window < 0) return -5;
  const int G = p.n_heads / p.n_kv_heads;
  const int GT = G == 1 ? 1 : G == 2 ? 2 : G == 8 ? 8 : 4;
  const int hgroups = (G + GT - 1) / GT;
  const int merge = p.splits == 1 ? MERGE_NONE : p.splits <= ATT_MAX_CLUSTER ? MERGE_CLUSTER : MERGE_GLOBAL;
  dim3 grid(p.n_kv_heads * hgroups, p.splits, p.batch), block(ATT_THREADS);
  dim3 cl(1, merge == MERGE_CLUSTER ? p.splits : 1, 1);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // K/V access mode: 1 "deep" (latency-bound launch: many loads in flight per thread), 2 "streamed" (the grid fills the GPU
  // several times over: pages come through a bulk-copy ring in shared memory), 0 plain register loads.  RLZ_ATT_MODE forces one.
  static const int mode_env = [] { const char* e = getenv("RLZ_ATT_MODE"); return e ? atoi(e) : -1; }();
  const long long ctas = (long long)grid.x * grid.y * grid.z;
  // 3 "tensor-core": bf16 cache, up to 8 splits, head_dim 64 / 80 / 96 / 128 - the default whenever it applies (measured against
  // the scalar modes: 7.7 vs 9.4 us at batch 1 x 640 tokens, 82 vs 114 us at batch 64 x 576, 217 vs 363 us at batch 64 x 2048 =
  // 0.94 of the measured copy bandwidth).  The scalar modes serve int8 caches, more than 8 splits and other head sizes.
  const bool mma_ok = merge != MERGE_GLOBAL && !p.kv_q8 && (p.head_dim == 64 || p.head_dim == 80 || p.head_dim == 96 || p.head_dim == 128);
  const int scalar_mode = ctas < 4LL * sms ? 1 : GT >= 4 ? 2 : 0;
  int mode = mma_ok ? 3 : scalar_mode;
  if (mode_env >= 0 && mode_env <= 3) mode = mode_env;
  if (mode == 3 && !mma_ok) mode = scalar_mode;
  if (mode == 3) {
    switch (GT) {
      case 1: return (int)launch_attn_mma_merge<1>(p, merge, grid, block, cl, st);
      case 2: return (int)launch_attn_mma_merge<2>(p, merge, grid, block, cl, st);
      case 8: return (int)launch_attn_mma_merge<8>(p, merge, grid, block, cl, st);
      default: return (int)launch_attn_mma_merge<4>(p, merge, grid, block, cl, st);
    }
  }
  const size_t ring = mode == 2 ? (size_t)ATT_RING * 4 * ATT_PAGE * (p.kv_q8 ? p.head_dim + 16 : 2 * p.head_dim) : 0;
#define RLZ_ATT_MODE_LAUNCH(GT_, M_, Q_) (mode == 1 ? launch_attn<GT_, M_, 1, Q_>(p, grid, block, cl, 0, st) \
                                        : mode == 2 ? launch_attn<GT_, M_, 2, Q_>(p, grid, block, cl, ring, st) \
                                                    : launch_attn<GT_, M_, 0, Q_>(p, grid, block, cl, 0, st))
#define RLZ_ATT_LAUNCH(GT_, M_) (p.kv_q8 ? RLZ_ATT_MODE_LAUNCH(GT_, M_, 1) : RLZ_ATT_MODE_LAUNCH(GT_, M_, 0))
#define RLZ_ATT_CASE(GT_) \
  (merge == MERGE_NONE ? RLZ_ATT_LAUNCH(GT_, MERGE_NONE) : merge == MERGE_CLUSTER ? RLZ_ATT_LAUNCH(GT_, MERGE_CLUSTER) : RLZ_ATT_LAUNCH(GT_, MERGE_GLOBAL))
  cudaError_t e;
  switch (GT) {
    case 1: e = RLZ_ATT_CASE(1); break;
    case 2: e = RLZ_ATT_CASE(2); break;
    case 8: e = RLZ_ATT_CASE(8); break;
    default: e = RLZ_ATT_CASE(4); break;
  }
#undef RLZ_ATT_LAUNCH
#undef RLZ_ATT_MODE_LAUNCH
#undef RLZ_ATT_CASE
  return (int)e;
}

}  // namespace rlz

extern "C" {

// scratch sizes for a launch configuration (floats / ints)
long long rlz_attn_decode_partial_floats(int batch, int n_heads, int splits, int head_dim) {
  return (long long)batch * n_heads * splits * (head_dim + 2);
}
long long rlz_attn_decode_counter_ints(int batch, int n_heads) { return (long long)batch * n_heads; }

int rlz_attn_decode(const rlz::AttnDecodeParams* pp, void* stream) { return rlz::attn_decode_dispatch(*pp, (cudaStream_t)stream); }

}  // extern "C"

// ---- allocation-free variant: scratch lives in the library image (see attn_decode_static.h) -----
namespace rlz {
static __device__ __align__(256) float g_static_partial[RLZ_ATTN_STATIC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) int32_t g_static_counters[RLZ_ATTN_STATIC_MAX_COUNTERS];

constexpr int STATIC_MAX_DEVICES = 64;
struct StaticScratch { float* partial; int32_t* counters; bool ready; };
static StaticScratch g_static_scratch[STATIC_MAX_DEVICES];
}  // namespace rlz

extern "C" {

const char* rlz_attn_decode_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case RLZ_STATIC_TOO_LARGE: return "attention launch needs more scratch than the built-in arrays hold (see attn_decode_static.h for the limits)";
    case RLZ_STATIC_NO_DEVICE: return "no current CUDA device, or its ordinal is beyond the supported range";
    default: return code < 0 ? "invalid attention parameters" : "CUDA error (see cudaGetErrorString)";
  }
}

int rlz_attn_decode_static(const rlz::AttnDecodeParams* pp, void* stream) {
  using namespace rlz;
  AttnDecodeParams p = *pp;
  if (p.head_dim % 8 || p.head_dim > 128 || p.head_dim < 8) return -1;
  if (p.n_kv_heads < 1 || p.n_heads % p.n_kv_heads || p.splits < 1 || p.batch < 1) return -2;
  if (p.rope_dim > p.head_dim || (p.rope_dim & 1)) return -3;
  if (((uintptr_t)p.k_cache & 15) || ((uintptr_t)p.v_cache & 15)) return -4;
  const long long need_f = (long long)p.batch * p.n_heads * p.splits * (p.head_dim + 2);
  const long long need_c = (long long)p.batch * p.n_heads;
  if (need_f > RLZ_ATTN_STATIC_MAX_PARTIAL_FLOATS || need_c > RLZ_ATTN_STATIC_MAX_COUNTERS) return RLZ_STATIC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) return RLZ_STATIC_NO_DEVICE;
  cudaStream_t st = (cudaStream_t)stream;
  StaticScratch& sc = g_static_scratch[dev];
  if (!sc.ready) {
    // In host code the array names are stand-ins; the device addresses come from the runtime,
    // once per device, with that device current.
    cudaError_t e = cudaGetSymbolAddress((void**)&sc.partial, g_static_partial);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress((void**)&sc.counters, g_static_counters);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemsetAsync(sc.counters, 0, sizeof(int32_t) * RLZ_ATTN_STATIC_MAX_COUNTERS, st);   // counters must start at zero
    if (e != cudaSuccess) return (int)e;
    sc.ready = true;
  }
  p.partial = sc.partial;
  p.counters = sc.counters;
  return attn_decode_dispatch(p, st);
}

// 0 / 3201 (a streamed K/V stage never arrived)
int rlz_attn_decode_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, rlz::g_attn_decode_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) { int z = 0; cudaMemcpyToSymbol(rlz::g_attn_decode_error, &z, sizeof(int)); }
  return v;
}

int rlz_sizeof_attn_decode_params() { return (int)sizeof(rlz::AttnDecodeParams); }

}  // extern "C"
