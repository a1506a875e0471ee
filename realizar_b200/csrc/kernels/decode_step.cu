// One decode step of a batch-1 sequence as ONE persistent cooperative kernel.
//
// The step is a short program of operations (embedding, fused-norm GEMVs, attention, argmax) that
// depend on one another through a few kilobytes of activations.  Launched one kernel per operation,
// each dependency costs a kernel boundary (drain, launch latency, cold prologue) - about 8 us against
// 4-6 us of weight streaming.  Here the grid stays resident (OCC CTAs per SM), every CTA walks the same
// program, and operations are separated by a grid-wide barrier in global memory (one atomic arrival per
// CTA, one polled generation word).  While a CTA waits, the weights of the operations after the next
// one are already on their way into L2 (prefetch two operations ahead), so HBM keeps streaming across
// the barriers.
//
// The operation bodies are the same device functions the one-launch-per-operation kernels use
// (gemv_body.cuh, attention_decode_body.cuh); attention jobs run on quarter-CTAs of 128 threads
// with named barriers and merge their context splits through global memory (last arrival merges).
//
// Every wait is bounded: a barrier that is not released within `spin_limit` polls records status 4001
// and the CTA leaves; the others run into the same limit and leave too.
//
// Serves the same purpose as the reference's CUDA-graph-captured decode and its persistent
// megakernel experiments (src/cuda/executor/layers/graphed_capture.rs:16-364,
// src/cuda/executor/layers/forward_graphed_decode.rs:18-211).
#include "common.cuh"
#include "../quant_blocks.h"
#include "gemv_body.cuh"
#include "attention_decode_body.cuh"
#include <math.h>

namespace rlz {

static_assert(sizeof(GemvParams) <= 1024 && sizeof(AttnDecodeParams) <= 1024, "parameter staging buffer too small");

enum { STEP_EMBED = 0, STEP_GEMV = 1, STEP_ATTN = 2, STEP_ARGMAX = 3 };
constexpr int STEP_PARAM_MAX = 1024;      // largest parameter block (the GEMV description), rounded up

struct StepOp {
  int32_t kind;
  int32_t grid;            // CTAs (GEMV), 128-thread jobs (attention), unused otherwise
  int64_t params;          // byte offset of the parameter struct in the program blob
};

struct StepEmbed {
  const uint8_t* table; const int32_t* tokens; const float* pos_table; const int32_t* positions; float* out;
  int64_t row_bytes;
  int32_t qtype, hidden, vocab, _pad;
};

struct StepArgmax {
  const float* logits; int32_t* out; float* out_val;
  int32_t vocab, index_offset;
};

struct StepProgram {
  const uint8_t* blob;     // device: StepOp[nops], then the parameter structs (16-byte aligned offsets)
  uint32_t* sync;          // device, 128 words on separate 128-byte lines: [0] barrier arrivals, [32] barrier generation, [64] argmax ticket, [96..97] argmax key
  int32_t* status;         // device: 0 while healthy
  int64_t spin_limit;      // polls of one barrier wait before giving up
  int32_t nops;
  int32_t occ;             // CTAs per SM the program was laid out for (1 or 2)
  int32_t attn_gt;         // query heads per attention job (1, 2 or 4)
  int32_t skip;            // diagnostics: bit 0 skip GEMV work, bit 1 skip attention work, bit 2 no weight prefetch (results are wrong)
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}

constexpr int SYNC_ARRIVE = 0, SYNC_GEN = 32, SYNC_TICKET = 64, SYNC_KEY = 96;     // word offsets, one 128-byte line each

__device__ __forceinline__ uint32_t atom_add_release_u32(uint32_t* p, uint32_t v) {
  uint32_t old; asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory"); return old;
}

// Grid-wide barrier (all CTAs are co-resident: cooperative launch).  `gen` is the generation this CTA has seen (thread 0).
// Arrival is one release-atomic per CTA, the wait an acquire-poll of the generation word (on its own cache line, so that the
// pollers do not slow the arrivals down).  Between its arrival and its wait a CTA does work that depends on nothing the other
// CTAs write (staging the next operation's parameters, weight prefetch).  The wait returns false when it ran out (a CTA that gives up
// leaves; the others then run into the same limit).
__device__ __forceinline__ void grid_barrier_arrive(const StepProgram& prog) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atom_add_release_u32(prog.sync + SYNC_ARRIVE, 1u);     // this CTA's writes are visible before its arrival
    if (old == gridDim.x - 1) {
      *(volatile uint32_t*)(prog.sync + SYNC_ARRIVE) = 0;                        // reset for the next barrier, then release everybody
      atom_add_release_u32(prog.sync + SYNC_GEN, 1u);
    }
  }
}
__device__ __forceinline__ bool grid_barrier_wait(const StepProgram& prog, uint32_t& gen, int* ok_s) {
  if (threadIdx.x == 0) {
    int ok = 1;
    int64_t spins = 0;
    while (ld_acquire_u32(prog.sync + SYNC_GEN) == gen) {
      if (++spins > prog.spin_limit) { ok = 0; atomicExch(prog.status, 4001); break; }
    }
    __threadfence();                                        // later reads of this CTA see the other CTAs' writes
    ++gen;
    *ok_s = ok;
  }
  __syncthreads();
  return *ok_s != 0;
}

// monotone map float -> uint32 (larger float, larger key)
__device__ __forceinline__ uint32_t step_float_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void step_embed(const StepEmbed& e, uint8_t* smem) {
  const int be = qtype_block_elems(e.qtype), bb = qtype_block_bytes(e.qtype);
  const int ce = be <= 1 ? 256 : be;                         // elements per chunk
  const int nchunks = (e.hidden + ce - 1) / ce;
  const int tok = e.tokens[0];
  float* tmp = (float*)smem;
  for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int i0 = c * ce, n = min(ce, e.hidden - i0);
    const bool valid = tok >= 0 && tok < e.vocab;
    const uint8_t* row = e.table + (int64_t)(valid ? tok : 0) * e.row_bytes;
    if (valid && be > 1) {
      if (threadIdx.x == 0) dequant_block(e.qtype, row + (int64_t)c * bb, tmp);
      __syncthreads();
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float v = 0.f;
      if (valid) {
        if (be > 1) v = tmp[i];
        else if (e.qtype == QT_F32) v = ((const float*)row)[i0 + i];
        else { const uint16_t h = ((const uint16_t*)row)[i0 + i]; v = e.qtype == QT_F16 ? half_bits_to_float(h) : bf16_bits_to_float(h); }
        if (e.pos_table) v += e.pos_table[(int64_t)e.positions[0] * e.hidden + i0 + i];
      }
      e.out[i0 + i] = v;
    }
    __syncthreads();
  }
}

// every CTA folds its slice into a 64-bit (value, smallest index) key; the last one to finish decodes it and cleans up
__device__ __forceinline__ void step_argmax(const StepArgmax& a, uint32_t* sync, uint8_t* smem) {
  float* sval = (float*)smem; int* sidx = (int*)(smem + 40 * 4);
  const int nsl = gridDim.x;
  const int per = ((a.vocab + nsl - 1) / nsl + 3) & ~3;
  const int i0 = blockIdx.x * per, i1 = min(a.vocab, i0 + per);
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) { const float v = a.logits[i]; if (v > best) { best = v; bi = i; } }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
  __syncthreads();
  if (threadIdx.x != 0) return;
  for (int w = 1; w < nw; ++w) if (sval[w] > best || (sval[w] == best && sidx[w] < bi)) { best = sval[w]; bi = sidx[w]; }
  unsigned long long* key = (unsigned long long*)(sync + SYNC_KEY);
  if (bi != 0x7fffffff) atomicMax(key, ((unsigned long long)step_float_key(best) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)bi));
  __threadfence();
  if (atomicAdd(&sync[SYNC_TICKET], 1u) != (unsigned)nsl - 1) return;
  __threadfence();
  const unsigned long long k = atomicExch(key, 0ull);
  sync[SYNC_TICKET] = 0;
  const uint32_t kv = (uint32_t)(k >> 32), idx = 0xFFFFFFFFu - (uint32_t)k;
  a.out[0] = (k ? (int)idx : 0) + a.index_offset;
  if (a.out_val) a.out_val[0] = k ? __uint_as_float((kv & 0x80000000u) ? (kv & 0x7FFFFFFFu) : ~kv) : -INFINITY;
}

template <int GT, int TBO>
__device__ __forceinline__ void step_attention(const AttnDecodeParams& p, int jobs, uint8_t* smem) {
  const int sub = threadIdx.x >> 7, tid = threadIdx.x & 127, nsub = blockDim.x >> 7;
  const int G = p.n_heads / p.n_kv_heads;
  const int gx = p.n_kv_heads * ((G + GT - 1) / GT);
  for (int j = blockIdx.x + sub * gridDim.x; j < jobs; j += gridDim.x * nsub) {     // job -> (head group, split, sequence)
    const int bz = j / (gx * p.splits), r = j - bz * gx * p.splits;
    const int by = r / gx, bx = r - by * gx;
    if (p.splits == 1) {
      AttnSmem<GT, MERGE_NONE>* sm = (AttnSmem<GT, MERGE_NONE>*)smem + sub;
      attn_decode_body<GT, MERGE_NONE, 0, 0, TBO, true>(p, bx, by, bz, tid, *sm, 1 + sub);
    } else {
      AttnSmem<GT, MERGE_GLOBAL>* sm = (AttnSmem<GT, MERGE_GLOBAL>*)smem + sub;
      attn_decode_body<GT, MERGE_GLOBAL, 0, 0, TBO, true>(p, bx, by, bz, tid, *sm, 1 + sub);
    }
    asm volatile("bar.sync %0, 128;" ::"r"(1 + sub) : "memory");      // the quarter is done with its shared memory
  }
}

template <int OCC, int GT>
__global__ void __launch_bounds__(GEMV_THREADS, OCC) decode_step_kernel(const __grid_constant__ StepProgram prog) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int ok_s;
  const StepOp* ops = (const StepOp*)prog.blob;
  uint32_t gen = threadIdx.x == 0 ? ld_acquire_u32(prog.sync + SYNC_GEN) : 0u;
  int pf_done = 0;                                              // operations up to this index have had their weights prefetched
  constexpr int TBO = OCC == 2 ? 2 : GT == 1 ? 8 : GT == 2 ? 6 : 4;
  // The operation records and their parameter blocks never change while the kernel runs.  Each is copied into shared
  // memory one operation ahead (before the barrier wait), so the dependent chain record -> parameters -> pointers
  // costs no global-memory round trips after the barrier.
  __shared__ __align__(16) uint8_t pbuf[2][STEP_PARAM_MAX];
  __shared__ StepOp opbuf[2];
  auto stage_op = [&](int i) {
    const StepOp o = ops[i];
    if (threadIdx.x == 0) opbuf[i & 1] = o;
    const int bytes = o.kind == STEP_GEMV ? (int)sizeof(GemvParams) : o.kind == STEP_ATTN ? (int)sizeof(AttnDecodeParams)
                    : o.kind == STEP_EMBED ? (int)sizeof(StepEmbed) : (int)sizeof(StepArgmax);
    const uint4* src = (const uint4*)(prog.blob + o.params);
    for (int j = threadIdx.x; j < (bytes + 15) / 16; j += blockDim.x) ((uint4*)pbuf[i & 1])[j] = __ldg(src + j);
  };
  stage_op(0);
  __syncthreads();
  for (int i = 0; i < prog.nops; ++i) {
    const int kind = opbuf[i & 1].kind, grid = opbuf[i & 1].grid;
    const uint8_t* pp = pbuf[i & 1];
    if (kind == STEP_GEMV) {
      if (prog.skip & 1) goto done;
      const GemvParams& p = *(const GemvParams*)pp;
      for (int v = blockIdx.x; v < grid; v += gridDim.x) {
        gemv_body<1, true, false>(p, v, smem);
        __syncthreads();
      }
    } else if (kind == STEP_ATTN) {
      if (!(prog.skip & 2)) step_attention<GT, TBO>(*(const AttnDecodeParams*)pp, grid, smem);
    } else if (kind == STEP_EMBED) {
      step_embed(*(const StepEmbed*)pp, smem);
    } else {
      step_argmax(*(const StepArgmax*)pp, prog.sync, smem);
    }
  done:
    if (i + 1 >= prog.nops) break;
    grid_barrier_arrive(prog);
    stage_op(i + 1);
    // weights of the operations up to two ahead start moving towards L2 before this CTA waits
    const int pf_to = min(i + 2, prog.nops - 1);
    for (int j = max(pf_done, i) + 1; j <= pf_to; ++j) {
      if (ops[j].kind != STEP_GEMV || (prog.skip & 4)) continue;
      const GemvParams& q = *(const GemvParams*)(prog.blob + ops[j].params);
      for (int v = blockIdx.x; v < ops[j].grid; v += gridDim.x) gemv_prefetch_slab(q, v);
    }
    pf_done = max(pf_done, pf_to);
    if (!grid_barrier_wait(prog, gen, &ok_s)) return;
  }
}

template <int OCC, int GT>
static cudaError_t launch_step(const StepProgram& prog, int sms, size_t smem, cudaStream_t st) {
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(decode_step_kernel<OCC, GT>, smem); e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(OCC * sms); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;              // all CTAs resident at once, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&cfg, decode_step_kernel<OCC, GT>, prog);
}

}  // namespace rlz

extern "C" {

// Shared memory one attention quarter-CTA needs for `gt` query heads per job.
int rlz_decode_step_attn_smem(int gt) {
  using namespace rlz;
  switch (gt) {
    case 1: return (int)sizeof(AttnSmem<1, MERGE_GLOBAL>);
    case 2: return (int)sizeof(AttnSmem<2, MERGE_GLOBAL>);
    case 4: return (int)sizeof(AttnSmem<4, MERGE_GLOBAL>);
    default: return -1;
  }
}

// Launch the program.  `smem` = dynamic shared memory per CTA (the largest GEMV staging area or four attention
// quarters, whichever is larger).  Returns 0, a negative code for an unsupported shape, or a positive cudaError_t
// (cudaErrorCooperativeLaunchTooLarge when the grid cannot be co-resident).
int rlz_decode_step(const rlz::StepProgram* pp, long long smem, void* stream) {
  using namespace rlz;
  const StepProgram& prog = *pp;
  if (prog.nops < 1 || !prog.blob || !prog.sync || !prog.status) return -1;
  if (prog.occ != 1 && prog.occ != 2) return -2;
  if (prog.occ == 2 && prog.attn_gt != 1) return -3;
  if (smem < 1024 || smem > 226 * 1024) return -4;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  cudaStream_t st = (cudaStream_t)stream;
  e = cudaMemsetAsync(prog.sync, 0, sizeof(uint32_t), st);   // barrier arrivals (word 0) start at zero even after an aborted step
  if (e != cudaSuccess) return (int)e;
  if (prog.occ == 2) return (int)launch_step<2, 1>(prog, sms, (size_t)smem, st);
  switch (prog.attn_gt) {
    case 1: return (int)launch_step<1, 1>(prog, sms, (size_t)smem, st);
    case 2: return (int)launch_step<1, 2>(prog, sms, (size_t)smem, st);
    case 4: return (int)launch_step<1, 4>(prog, sms, (size_t)smem, st);
    default: return -3;
  }
}

int rlz_sizeof_step_program() { return (int)sizeof(rlz::StepProgram); }
int rlz_sizeof_step_op() { return (int)sizeof(rlz::StepOp); }
int rlz_sizeof_step_embed() { return (int)sizeof(rlz::StepEmbed); }
int rlz_sizeof_step_argmax() { return (int)sizeof(rlz::StepArgmax); }

}  // extern "C"
