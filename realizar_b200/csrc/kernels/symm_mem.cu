// Symmetric peer memory for tensor parallelism: every rank allocates a buffer, exports a CUDA IPC
// handle, and maps the buffers of the other ranks of the node, so kernels can store into and load
// from a peer's memory over NVLink.  Also the small kernels that go with the in-kernel
// collectives: the per-step epoch counter and the exchange of per-rank argmax candidates.
//
// The reference has no communication backend (its Communicator is a single-process mock,
// src/parallel/mod_all_reduce_communicator.rs:2-110); this is the node-local real one.
#include "common.cuh"
#include "gemv_params.h"
#include <cstring>

namespace rlz {

__global__ void epoch_bump_kernel(uint32_t* epoch) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *epoch += 1;
}

// x[t, j] += sum over all writers (ranks x K splits) of the value pushed into this rank's inbox for (t, j) at call site
// `site`; every element is polled until its tag matches (bounded; on expiry status = 2003 and the element contributes
// what was read).  Buffer and tag follow the GEMM epilogue: buffer = (epoch * nsites + site) & 1, tag = epoch * 256 + site.
__global__ void ll_reduce_kernel(const uint2* inbox, const uint32_t* epoch_p, int32_t* status, int64_t spin_limit, int writers, int rows_cap,
                                 int64_t row_pairs, int site, int nsites, int n, float* x, int64_t ldx) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const uint32_t epoch = *epoch_p;
  const uint32_t tag = epoch * 256u + (uint32_t)site;
  const int64_t buf = (int64_t)((epoch * (uint32_t)nsites + (uint32_t)site) & 1u) * writers;
  const uint2* base = inbox + buf * rows_cap * row_pairs + (int64_t)t * row_pairs + j;
  float v = 0.f;
  for (int q = 0; q < writers; ++q) {
    const uint2* src = base + (int64_t)q * rows_cap * row_pairs;
    uint2 w = ld_pair_sys(src);
    for (int64_t spins = 0; w.y != tag; ++spins) {
      if (spins > spin_limit) { atomicExch(status, 2003); break; }
      w = ld_pair_sys(src);
    }
    v += __uint_as_float(w.x);
  }
  x[(int64_t)t * ldx + j] += v;
}

struct CandExchange {                 // all-gather of one (value, index) pair per batch row and rank
  uint2* inbox[GEMV_AR_MAX_RANKS];    // rank r's inbox: [parity 2][rank][batch][2] pairs {payload, epoch}
  const uint32_t* epoch;
  int32_t* status;
  int64_t spin_limit;
  int32_t rank, world, batch, max_batch;
};

__device__ __forceinline__ void cx_store(uint2* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 cx_load(const uint2* p) {
  uint2 v; asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory"); return v;
}

// in: local (value, token id) per batch row; out: the pair with the largest value over all ranks
// (ties -> smallest token id).  One CTA, one thread per batch row; same epoch-tagged 8-byte stores
// as the GEMV all-reduce, so no fences or flags.
__global__ void cand_exchange_kernel(const __grid_constant__ CandExchange c, const float* val, const int32_t* idx, int32_t* out_idx, float* out_val) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = *c.epoch;
  const int b = threadIdx.x;
  if (b >= c.batch) return;
  const int64_t slot = (int64_t)c.max_batch * 2;
  const int64_t base = (int64_t)(epoch & 1u) * c.world * slot;
  for (int q = 0; q < c.world; ++q) {
    uint2* dst = c.inbox[q] + base + (int64_t)c.rank * slot + 2 * b;
    cx_store(dst, __float_as_uint(val[b]), epoch);
    cx_store(dst + 1, (uint32_t)idx[b], epoch);
  }
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int q = 0; q < c.world; ++q) {
    const uint2* src = c.inbox[c.rank] + base + (int64_t)q * slot + 2 * b;
    uint2 v = cx_load(src), i = cx_load(src + 1);
    for (int64_t spins = 0; v.y != epoch || i.y != epoch; ++spins) {
      if (spins > c.spin_limit) { atomicExch(c.status, 2002); break; }
      v = cx_load(src); i = cx_load(src + 1);
    }
    const float fv = __uint_as_float(v.x); const int ii = (int)i.x;
    if (fv > best || (fv == best && ii < bi)) { best = fv; bi = ii; }
  }
  out_idx[b] = bi;
  if (out_val) out_val[b] = best;
}

}  // namespace rlz

extern "C" {
using namespace rlz;

// Allocate `bytes` of zeroed device memory that other processes can map; writes the 64-byte IPC handle.
int rlz_symm_alloc(unsigned long long bytes, void** ptr, void* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int rlz_symm_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int rlz_symm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
int rlz_symm_free(void* ptr) { return (int)cudaFree(ptr); }

int rlz_epoch_bump(uint32_t* epoch, void* stream) {
  return (int)launch(epoch_bump_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, epoch);
}

int rlz_ll_reduce(const void* inbox, const uint32_t* epoch, int32_t* status, long long spin_limit, int writers, int rows_cap, long long row_pairs,
                  int site, int nsites, int tokens, int n, float* x, long long ldx, void* stream) {
  if (tokens < 1 || tokens > rows_cap || n < 1 || n > row_pairs || writers < 1 || writers > 64 || site < 0 || site >= nsites || site >= 256) return -1;
  return (int)launch(ll_reduce_kernel, dim3((n + 255) / 256, tokens), dim3(256), 0, (cudaStream_t)stream, (const uint2*)inbox, epoch, status,
                     (int64_t)spin_limit, writers, rows_cap, (int64_t)row_pairs, site, nsites, n, x, (int64_t)ldx);
}

int rlz_cand_exchange(const CandExchange* c, const float* val, const int32_t* idx, int32_t* out_idx, float* out_val, void* stream) {
  if (c->batch < 1 || c->batch > c->max_batch || c->max_batch > 1024 || c->world < 1 || c->world > GEMV_AR_MAX_RANKS) return -1;
  const int threads = (c->batch + 31) / 32 * 32;
  return (int)launch(cand_exchange_kernel, dim3(1), dim3(threads), 0, (cudaStream_t)stream, *c, val, idx, out_idx, out_val);
}

int rlz_sizeof_cand_exchange() { return (int)sizeof(rlz::CandExchange); }

}  // extern "C"
