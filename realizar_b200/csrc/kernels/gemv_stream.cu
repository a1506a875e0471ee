// Streamed decode GEMV for K-quant weights (Q4_K / Q5_K / Q6_K), batch 1..4.
//
// A CTA owns a contiguous slab of weight rows.  One thread drives a ring of shared-memory stages
// that the TMA engine fills with `cp.async.bulk` (completion on an mbarrier); the first stages
// are requested before the kernel waits for its predecessor (programmatic dependent launch), so
// weight bytes are already in flight while the previous kernel drains.  Two lanes then consume
// one 256-weight block per stage from shared memory, half a block each (csrc/gemv_blocks.h): the
// scale decode is paid once per 128 weights and the global-memory access pattern is a plain
// linear stream.
// Prologue (norm + int8 staging of the input) and epilogue (bias / activation / gated combine /
// second accumulated matrix / residual) are those of the register-path kernel in gemv.cu, which
// remains the path for the 32-wide block types.
//
// Every mbarrier wait is bounded: if a stage does not arrive the CTA records an error code in
// g_rlz_error, skips the math of that stage and finishes normally.
//
// Replaces the same reference kernels as gemv.cu (src/cuda/executor/q4k_mwv_gemv.rs:7-945).
#include "common.cuh"
#include <stdlib.h>
#include "../gemv_blocks.h"
#include "gemv_common.cuh"

namespace rlz {

constexpr int GS_THREADS = 512;
constexpr int GS_BLOCKS = GS_THREADS / 2;        // weight blocks per stage
constexpr int GS_MAX_STAGES = 4;
constexpr uint32_t GS_WAIT_LIMIT = 1u << 22;      // try_wait iterations before giving up (~0.1-1 s)

__device__ int g_rlz_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// int8 staging in the chunk-major ActBlk layout (see gemv_blocks.h)
template <int B>
__device__ void stage_x_blk(const GemvX& X, int8_t* xq, uint32_t* rec4, float* rec6, float* red) {
  const int k = X.k, nsb = k >> 8;
#pragma unroll 1
  for (int b = 0; b < B; ++b) {
    const float* x = X.x + (int64_t)b * X.ld;
    float mean, rstd;
    row_stats(X, x, red, &mean, &rstd);
    for (int base = (threadIdx.x & ~31) * 4; base < k; base += blockDim.x * 4) {   // warp-uniform bound
      const int i = base + (threadIdx.x & 31) * 4;
      const bool ok = i < k;
      float4 v = ok ? load_normed(X, x, i, mean, rstd) : make_float4(0.f, 0.f, 0.f, 0.f);
      float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float d = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
      const int q0 = __float2int_rn(v.x * inv), q1 = __float2int_rn(v.y * inv), q2 = __float2int_rn(v.z * inv), q3 = __float2int_rn(v.w * inv);
      int s16 = q0 + q1 + q2 + q3;
      s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
      s16 += __shfl_xor_sync(0xffffffffu, s16, 2);
      const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 4);
      if (ok) {
        const int sb = i >> 8, c = (i >> 4) & 15;
        *(uint32_t*)(xq + (int64_t)b * k + blk_chunk_off(nsb, sb, c) + (i & 15)) =
            (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
        if ((threadIdx.x & 3) == 0) {
          float* r6 = rec6 + ((int64_t)b * (k >> 4) + c * nsb + sb) * 2;
          r6[0] = d; r6[1] = d * (float)s16;
        }
        if ((threadIdx.x & 7) == 0) {
          const int j = (i >> 5) & 7;
          uint32_t* r4 = rec4 + ((int64_t)b * (k >> 6) + (j >> 1) * nsb + sb) * 4 + (j & 1);
          r4[0] = __float_as_uint(d); r4[2] = __float_as_uint(d * (float)s32);
        }
      }
    }
  }
}

struct StageDesc { int seg; int blk0; int nblk; };     // blocks [blk0, blk0+nblk) of the segment's slab

template <int B>
__global__ void __launch_bounds__(GS_THREADS, 1) gemv_stream_kernel(const __grid_constant__ GemvParams p, int nstage, int stage_bytes) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[GS_MAX_STAGES];
  __shared__ int failed;
  int m = 0;
  while (m + 1 < p.nmat && (int)blockIdx.x >= p.mat[m + 1].cta_begin) ++m;
  const GemvMat& M = p.mat[m];
  const int r0 = ((int)blockIdx.x - M.cta_begin) * M.rows_per_cta;
  const int r1 = min(M.n, r0 + M.rows_per_cta);
  const int nrows = r1 - r0;
  const int tid = threadIdx.x;

  // stage bookkeeping: segment s contributes ceil(nrows * nsb_s / GS_BLOCKS) stages
  int nsb[2], bb[2], nst[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    nsb[s] = s < M.nseg ? M.seg[s].k >> 8 : 0;
    bb[s] = s < M.nseg ? dev_block_bytes(M.seg[s].qtype) : 0;
    nst[s] = (nrows * nsb[s] + GS_BLOCKS - 1) / GS_BLOCKS;
  }
  const int total_stages = nst[0] + nst[1];
  auto describe = [&](int st) {
    StageDesc dsc;
    dsc.seg = st < nst[0] ? 0 : 1;
    const int ls = st - (dsc.seg ? nst[0] : 0);
    dsc.blk0 = ls * GS_BLOCKS;
    dsc.nblk = min(GS_BLOCKS, nrows * nsb[dsc.seg] - dsc.blk0);
    return dsc;
  };
  uint8_t* ring = smem;                                   // nstage * stage_bytes
  auto issue = [&](int st) {                              // called by thread 0 only
    const StageDesc dsc = describe(st);
    const int slot = st % nstage;
    const uint32_t bytes = (uint32_t)dsc.nblk * (uint32_t)bb[dsc.seg];
    const uint8_t* src = M.seg[dsc.seg].W + (int64_t)r0 * M.seg[dsc.seg].stride + (int64_t)dsc.blk0 * bb[dsc.seg];
    mbar_expect_tx(&full[slot], bytes);
    bulk_g2s(ring + (size_t)slot * stage_bytes, src, bytes, &full[slot]);
  };

  if (tid == 0) {
    failed = 0;
    for (int i = 0; i < nstage; ++i) mbar_init(&full[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (tid == 0) {                                         // weights do not depend on earlier kernels:
    for (int st = 0; st < min(nstage, total_stages); ++st) issue(st);   // request them before the dependency wait
  }
  pdl_launch_dependents();
  pdl_wait();

  // shared memory carve-up behind the ring
  const int kq = p.max_k;
  uint8_t* actbase = smem + (size_t)nstage * stage_bytes;
  int8_t* xq = (int8_t*)actbase;
  uint32_t* rec4 = (uint32_t*)(actbase + (size_t)B * kq);             // B * kq/64 records of 16 bytes
  float* rec6 = (float*)(rec4 + (size_t)B * (kq >> 6) * 4);           // B * kq/16 records of 8 bytes
  float* red = rec6 + (size_t)B * (kq >> 4) * 2;
  float* blocksum = red + 40;                             // [2][GS_THREADS][B]
  float* rowacc = blocksum + 2 * GS_THREADS * B;          // [max_rows][2][B]
  // lanes 0-15 of a warp take the first halves of 16 consecutive blocks, lanes 16-31 the second
  // halves: every group of 8 lanes then reads consecutive addresses (no bank conflicts)
  const int lane = tid & 31, my_blk = (tid >> 5) * 16 + (lane & 15), my_half = lane >> 4;
  for (int i = tid; i < nrows * 2 * B; i += GS_THREADS) rowacc[i] = 0.f;

  int staged = -1;
  int st = 0;                                             // running stage number over both segments
  for (int seg = 0; seg < M.nseg; ++seg) {
    const GemvSeg& S = M.seg[seg];
    const int nsbs = nsb[seg], bbs = bb[seg], seg_blocks = nrows * nsbs;
    // all per-stage index arithmetic is incremental: the only divisions are these, once per segment
    const int q_step = GS_BLOCKS / nsbs, r_step = GS_BLOCKS - q_step * nsbs;
    int sb_my = my_blk % nsbs;                            // super-block index of my block inside its row
    int first_row = 0, first_rem = 0;                     // stage start = first_row * nsbs + first_rem
    if (S.x_id != staged) {
      __syncthreads();
      const GemvX& X = p.xs[S.x_id];
      if (X.k <= STAGE_MAXV * 4 * GS_THREADS) {
        const int k = X.k, nsbx = k >> 8;
        stage_rows_regs<B, true>(X, red,
          [&](int b, int i, uint32_t packed, float d, int s16, int s32) {
            const int sb = i >> 8, c = (i >> 4) & 15;
            *(uint32_t*)(xq + (int64_t)b * k + blk_chunk_off(nsbx, sb, c) + (i & 15)) = packed;
            if ((threadIdx.x & 3) == 0) {
              float* r6 = rec6 + ((int64_t)b * (k >> 4) + c * nsbx + sb) * 2;
              r6[0] = d; r6[1] = d * (float)s16;
            }
            if ((threadIdx.x & 7) == 0) {
              const int j = (i >> 5) & 7;
              uint32_t* r4 = rec4 + ((int64_t)b * (k >> 6) + (j >> 1) * nsbx + sb) * 4 + (j & 1);
              r4[0] = __float_as_uint(d); r4[2] = __float_as_uint(d * (float)s32);
            }
          },
          [](int, int, float4) {});
      } else stage_x_blk<B>(X, xq, rec4, rec6, red);
      staged = S.x_id;
      __syncthreads();
    }
    const ActBlk a{xq, (const U4*)rec4, (const F2*)rec6, S.k, nsbs};
    for (int blk0 = 0; blk0 < seg_blocks; blk0 += GS_BLOCKS, ++st) {
      const int nblk = min(GS_BLOCKS, seg_blocks - blk0);
      const int slot = st % nstage;
      const uint32_t parity = (uint32_t)(st / nstage) & 1u;
      bool arrived = false;
      for (uint32_t spin = 0; spin < GS_WAIT_LIMIT; ++spin) {
        if (mbar_try_wait(&full[slot], parity)) { arrived = true; break; }
      }
      if (!arrived) { failed = 1; atomicExch(&g_rlz_error, 1001); }
      float t[B];
#pragma unroll
      for (int b = 0; b < B; ++b) t[b] = 0.f;
      if (arrived && my_blk < nblk) {
        const uint8_t* blk = ring + (size_t)slot * stage_bytes + (size_t)my_blk * bbs;
        switch (S.qtype) {
          case QT_Q4_K: halfblock_dot<QT_Q4_K, B>(blk, sb_my, my_half, a, t); break;
          case QT_Q5_K: halfblock_dot<QT_Q5_K, B>(blk, sb_my, my_half, a, t); break;
          default: halfblock_dot<QT_Q6_K, B>(blk, sb_my, my_half, a, t); break;
        }
      }
      float* bs = blocksum + (size_t)(st & 1) * GS_THREADS * B;
#pragma unroll
      for (int b = 0; b < B; ++b) bs[(my_blk * 2 + my_half) * B + b] = t[b];
      __syncthreads();                                    // stage consumed, block sums visible
      if (tid == 0 && st + nstage < total_stages) issue(st + nstage);
      // fold the block sums of this stage into their rows (one thread per (row, batch) pair)
      for (int idx = tid;; idx += GS_THREADS) {
        const int rr = idx / B, b = idx - rr * B, row = first_row + rr;
        const int row_lo = row * nsbs;
        if (row >= nrows || row_lo >= blk0 + nblk) break;
        const int lo = max(row_lo, blk0) - blk0, hi = min(row_lo + nsbs, blk0 + nblk) - blk0;
        float v = 0.f;
        for (int j = 2 * lo; j < 2 * hi; ++j) v += bs[j * B + b];
        rowacc[(row * 2 + seg) * B + b] += v;
      }
      sb_my += r_step; if (sb_my >= nsbs) sb_my -= nsbs;
      first_row += q_step; first_rem += r_step;
      if (first_rem >= nsbs) { first_rem -= nsbs; ++first_row; }
    }
  }
  __syncthreads();
  gemv_epilogue<B>(p, M, rowacc, r0, r1);
}

size_t gs_fixed_smem(const GemvParams& p) {               // everything behind the ring
  const size_t B = (size_t)p.batch, kq = (size_t)p.max_k;
  return B * kq + B * (kq >> 6) * 16 + B * (kq >> 4) * 8 + 40 * 4 + 2 * GS_THREADS * B * 4 + (size_t)p.max_rows * 2 * B * 4;
}

template <int B>
cudaError_t launch_gs(const GemvParams& p, int grid, int nstage, int stage_bytes, cudaStream_t stream) {
  const size_t smem = (size_t)nstage * stage_bytes + gs_fixed_smem(p);
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(gemv_stream_kernel<B>, smem, 0); e != cudaSuccess) return e;
  return launch(gemv_stream_kernel<B>, dim3(grid), dim3(GS_THREADS), smem, stream, p, nstage, stage_bytes);
}

}  // namespace rlz

extern "C" {

// 0 / last error code recorded by a kernel of this library (1001: a GEMV weight stage never arrived)
int rlz_device_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, rlz::g_rlz_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) { int z = 0; cudaMemcpyToSymbol(rlz::g_rlz_error, &z, sizeof(int)); }
  return v;
}

// Same parameter block and return convention as rlz_gemv; every segment must be Q4_K / Q5_K / Q6_K
// with k % 256 == 0, rows contiguous (stride == row bytes).  Returns -20 when the launch does not
// qualify (the caller then uses rlz_gemv).
int rlz_gemv_stream(const rlz::GemvParams* pp, void* stream) {
  using namespace rlz;
  GemvParams p = *pp;
  if (p.nmat < 1 || p.nmat > GEMV_MAX_MATS || p.batch < 1 || p.batch > 4) return -1;
  int grid = 0, max_rows = 0, max_k = 0, max_bb = 0;
  for (int m = 0; m < p.nmat; ++m) {
    GemvMat& M = p.mat[m];
    if (M.nseg < 1 || M.nseg > 2 || M.n < 1 || M.rows_per_cta < 1) return -2;
    for (int s = 0; s < M.nseg; ++s) {
      const GemvSeg& S = M.seg[s];
      const int bbs = dev_block_bytes(S.qtype);
      if (bbs == 0 || S.k % 256) return -20;
      if (S.stride != (int64_t)(S.k / 256) * bbs) return -20;
      if (S.x_id < 0 || S.x_id >= GEMV_MAX_X || p.xs[S.x_id].k != S.k) return -4;
      if (((uintptr_t)S.W & 15)) return -5;
      if (S.k > max_k) max_k = S.k;
      if (bbs > max_bb) max_bb = bbs;
    }
    M.cta_begin = grid;
    grid += (M.n + M.rows_per_cta - 1) / M.rows_per_cta;
    if (M.rows_per_cta > max_rows) max_rows = M.rows_per_cta;
  }
  p.max_k = max_k; p.max_rows = max_rows; p.any_generic = 0;
  if (p.ar.enabled && (p.nmat != 1 || p.ar.world < 1 || p.ar.world > GEMV_AR_MAX_RANKS || p.mat[0].out_off != 0 || p.mat[0].n > p.ar.n)) return -8;
  const int stage_bytes = GS_BLOCKS * max_bb;
  const size_t fixed = gs_fixed_smem(p);
  const size_t budget = 227 * 1024 - 2048;                // leave room for static shared memory
  if (fixed + 2 * (size_t)stage_bytes > budget) return -20;
  int nstage = (int)((budget - fixed) / stage_bytes);
  if (nstage > GS_MAX_STAGES) nstage = GS_MAX_STAGES;
  // fewer stages = less shared memory per CTA, so that the CTAs of the next launch can become resident (and request their
  // weights) while this launch still runs; RLZ_GS_STAGES caps the ring depth
  static const int stage_cap = [] { const char* e = getenv("RLZ_GS_STAGES"); return e ? atoi(e) : 0; }();
  if (stage_cap >= 2 && nstage > stage_cap) nstage = stage_cap;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  switch (p.batch) {
    case 1: e = launch_gs<1>(p, grid, nstage, stage_bytes, st); break;
    case 2: e = launch_gs<2>(p, grid, nstage, stage_bytes, st); break;
    case 3: e = launch_gs<3>(p, grid, nstage, stage_bytes, st); break;
    default: e = launch_gs<4>(p, grid, nstage, stage_bytes, st); break;
  }
  return (int)e;
}

}  // extern "C"
