// Symmetric peer memory for tensor parallelism: every rank allocates a buffer, exports a CUDA IPC
// handle, and maps the buffers of the other ranks of the node, so kernels can store into and load
// from a peer's memory over NVLink.  Also the small kernels that go with the in-kernel
// collectives: the per-step epoch counter and the exchange of per-rank argmax candidates.
//
// The reference has no communication backend (its Communicator is a single-process mock,
// src/parallel/mod_all_reduce_communicator.rs:2-110); this is the node-local real one.
#include "common.cuh"
#include "gemv_params.h"
#include <cuda_bf16.h>
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

// ---- two-shot all-reduce of a row-parallel GEMM, second half -------------------------------------------------------------
// The GEMM epilogues of all ranks have stored their partial tiles of token row t into the inbox of the rank that OWNS t
// (t / own_rows) and published one tag per tile.  Here every owner, one CTA per owned row:
//   1. waits (bounded, one flag per thread) for the tiles that cover its row from every writer and K split;
//   2. sums them in writer order onto the fp32 residual row (which only the owner keeps up to date between layers);
//   3. applies the NEXT layer's norm and stores the bf16 row into the operand buffer `xb` of EVERY rank (all-gather by peer
//      stores), or, at the last site of a pass, sends the fp32 row itself to every rank (`push_x`);
//   4. fences and publishes the row's tag in every rank's all-gather flag array.
// CTA 0 then waits until the rows of all owners have arrived here, so that "this kernel has finished" means "xb / x are
// complete on this rank": the next GEMM reads them from LOCAL memory through TMA with no further synchronisation.
// Per rank and message this moves 2 * (world - 1) / world of the data instead of (world - 1) * 2 with the one-shot push.
struct RsReduce {
  const float* inbox;                  // this rank's reduce-scatter inbox
  const uint32_t* flags;               // this rank's tile flags
  uint32_t* ag_flags[GEMV_AR_MAX_RANKS];       // all-gather flags of every rank: [world owners][own_cap]
  __nv_bfloat16* xb[GEMV_AR_MAX_RANKS];        // operand buffer of every rank (null entries: no bf16 output at this site)
  float* xpeer[GEMV_AR_MAX_RANKS];             // residual stream of every rank (used with push_x)
  float* x;                            // local residual stream
  const float* nw; const float* nb;    // norm weight / bias of the norm that follows (may be null)
  const uint32_t* epoch; int32_t* status;
  int64_t spin_limit, ldx, ldxb, ld_in;
  int32_t rank, world, splits_stride, splits_used, rows_cap, own_rows, own_cap, tokens, n, nt, n_tiles, ntiles_cap, mtiles_cap;
  int32_t site, nsites, norm, push_x, wait_ag;
  float eps;
  int32_t _pad;
};

constexpr int RS_THREADS = 256, RS_MAXV = 8;      // n <= RS_MAXV * 4 * RS_THREADS = 8192

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ bool rs_poll(const uint32_t* f, uint32_t tag, int64_t limit) {
  for (int64_t spins = 0; spins <= limit; ++spins)
    if (ld_acquire_sys(f) == tag) return true;
  return false;
}

__global__ void __launch_bounds__(RS_THREADS) rs_reduce_kernel(const __grid_constant__ RsReduce c) {
  __shared__ float red[2 * RS_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t epoch = *c.epoch;
  const uint32_t tag = epoch * 256u + (uint32_t)c.site;
  const int64_t par = (int64_t)((epoch * (uint32_t)c.nsites + (uint32_t)c.site) & 1u);
  const int mine = max(0, min(c.own_rows, c.tokens - c.rank * c.own_rows));     // rows this rank owns in this call
  const int lt = (int)blockIdx.x;
  if (lt < mine) {
    const int t = c.rank * c.own_rows + lt;
    // 1. the tiles that cover row t: every writer, every K split, every feature tile of token tile t / nt
    const int nflags = c.world * c.splits_used * c.n_tiles, mt = t / c.nt;
    bool ok = true;
    for (int idx = tid; idx < nflags; idx += RS_THREADS) {
      const int w = idx / (c.splits_used * c.n_tiles), rem = idx - w * (c.splits_used * c.n_tiles);
      const int z = rem / c.n_tiles, i = rem - z * c.n_tiles;
      const uint32_t* f = c.flags + (((par * c.world + w) * c.splits_stride + z) * c.ntiles_cap + i) * c.mtiles_cap + mt;
      if (!rs_poll(f, tag, c.spin_limit)) ok = false;
    }
    if (!ok) atomicExch(c.status, 2004);
    __syncthreads();
    // 2. residual row + partial rows, in writer order (identical on every call: deterministic)
    float4 v[RS_MAXV];
    float* xrow = c.x + (int64_t)t * c.ldx;
#pragma unroll
    for (int it = 0; it < RS_MAXV; ++it) {
      const int f = (it * RS_THREADS + tid) * 4;
      v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (f < c.n) {
        float4 a = *(const float4*)(xrow + f);
        for (int w = 0; w < c.world; ++w)
          for (int z = 0; z < c.splits_used; ++z) {
            const float4 b = __ldcg((const float4*)(c.inbox + (((par * c.world + w) * c.splits_stride + z) * c.rows_cap + lt) * c.ld_in + f));
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
          }
        v[it] = a;
        *(float4*)(xrow + f) = a;
        if (c.push_x)
          for (int q = 0; q < c.world; ++q)
            if (q != c.rank) *(float4*)(c.xpeer[q] + (int64_t)t * c.ldx + f) = a;
      }
    }
    // 3. the norm that follows, bf16, to every rank's operand buffer
    if (c.xb[c.rank]) {
      float mean = 0.f, rstd = 1.f;
      if (c.norm != NORM_NONE) {
        if (c.norm == NORM_LAYER) {
          float s = 0.f;
#pragma unroll
          for (int it = 0; it < RS_MAXV; ++it) s += v[it].x + v[it].y + v[it].z + v[it].w;      // padding is zero
          s = warp_sum(s);
          if (lane == 0) red[warp] = s;
          __syncthreads();
          float tsum = 0.f;
#pragma unroll
          for (int w = 0; w < RS_THREADS / 32; ++w) tsum += red[w];
          mean = tsum / (float)c.n;
        }
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < RS_MAXV; ++it) {
          const bool in = (it * RS_THREADS + tid) * 4 < c.n;
          const float a = v[it].x - mean, b = v[it].y - mean, d = v[it].z - mean, e = v[it].w - mean;
          ss += in ? a * a + b * b + d * d + e * e : 0.f;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[RS_THREADS / 32 + warp] = ss;
        __syncthreads();
        float tsum = 0.f;
#pragma unroll
        for (int w = 0; w < RS_THREADS / 32; ++w) tsum += red[RS_THREADS / 32 + w];
        rstd = rsqrtf(tsum / (float)c.n + c.eps);
      }
#pragma unroll
      for (int it = 0; it < RS_MAXV; ++it) {
        const int f = (it * RS_THREADS + tid) * 4;
        if (f < c.n) {
          float4 a = v[it];
          if (c.norm != NORM_NONE) {
            a.x = (a.x - mean) * rstd; a.y = (a.y - mean) * rstd; a.z = (a.z - mean) * rstd; a.w = (a.w - mean) * rstd;
            if (c.nw) { const float4 g = __ldg((const float4*)(c.nw + f)); a.x *= g.x; a.y *= g.y; a.z *= g.z; a.w *= g.w; }
            if (c.nb) { const float4 g = __ldg((const float4*)(c.nb + f)); a.x += g.x; a.y += g.y; a.z += g.z; a.w += g.w; }
          }
          const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
          const uint2 packed = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
          for (int q = 0; q < c.world; ++q) *(uint2*)(c.xb[q] + (int64_t)t * c.ldxb + f) = packed;
        }
      }
    }
    __syncthreads();
    // 4. this row is complete everywhere: fence, then its tag to every rank
    if (tid == 0) {
      __threadfence_system();
      for (int q = 0; q < c.world; ++q)
        asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(c.ag_flags[q] + (int64_t)c.rank * c.own_cap + lt), "r"(tag) : "memory");
    }
  }
  if (blockIdx.x == 0 && c.wait_ag) {
    bool ok = true;
    for (int idx = tid; idx < c.tokens; idx += RS_THREADS) {
      const int o = idx / c.own_rows, l = idx - o * c.own_rows;
      if (!rs_poll(c.ag_flags[c.rank] + (int64_t)o * c.own_cap + l, tag, c.spin_limit)) ok = false;
    }
    if (!ok) atomicExch(c.status, 2005);
  }
}

}  // namespace rlz

extern "C" {
using namespace rlz;

// Owner-side half of the two-shot all-reduce (see rs_reduce_kernel).  Returns 0, -1 for invalid geometry or a cudaError_t.
int rlz_rs_reduce(const RsReduce* c, void* stream) {
  if (c->world < 1 || c->world > GEMV_AR_MAX_RANKS || c->rank < 0 || c->rank >= c->world || c->n < 4 || c->n % 4 || c->n > RS_MAXV * 4 * RS_THREADS) return -1;
  if (c->tokens < 1 || c->own_rows < 1 || c->own_rows > c->own_cap || c->own_rows > c->rows_cap || (long long)c->own_rows * c->world < c->tokens) return -1;
  if (c->splits_used < 1 || c->splits_used > c->splits_stride || c->n_tiles < 1 || c->n_tiles > c->ntiles_cap || c->nt < 1 ||
      (c->tokens + c->nt - 1) / c->nt > c->mtiles_cap || c->site < 0 || c->site >= 256 || c->site >= c->nsites) return -1;
  if ((c->ldx % 4) || (c->ldxb % 4) || (c->ld_in % 4)) return -1;
  const int mine = c->tokens - c->rank * c->own_rows;
  const int grid = mine < 1 ? 1 : (mine > c->own_rows ? c->own_rows : mine);
  return (int)launch(rs_reduce_kernel, dim3(grid), dim3(RS_THREADS), 0, (cudaStream_t)stream, *c);
}
int rlz_sizeof_rs_reduce() { return (int)sizeof(rlz::RsReduce); }

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
