// Dequant-GEMM on the 5th-generation tensor cores: Y[M, N] (+)= X[M, K] . W[N, K]^T with W in a
// K-quant block layout (Q4_K / Q5_K / Q6_K) or dense bf16/f16, X in bf16, fp32 accumulation in
// tensor memory.  Used for prefill and for decode batches too large for the GEMV kernels.
//
// One CTA owns 128 weight rows x NT tokens (x one K split) and is warp-specialised:
//   * warps 0-7 (256 threads) dequantise: per K step of 64 columns each thread turns 32 weights of
//     "its" row into bf16 and stores them into shared memory in the K-major 128-byte-swizzled
//     layout that tcgen05.mma reads (operand A);
//   * warp 8 (one thread) streams the activations (operand B, NT x 64 bf16) with TMA
//     (cp.async.bulk.tensor, 128-byte swizzle, zero fill beyond the last token);
//   * warp 9 (one thread) issues four tcgen05.mma (M=128, N=NT, K=16) per K step and commits them
//     to the stage's "empty" mbarrier;
//   * a ring of GM_STAGES shared-memory stages decouples the three roles ("full" barrier: 8 warp
//     arrivals + the TMA transaction bytes; "empty" barrier: the MMA commit);
//   * the accumulator lives in TMEM (NT columns); after the last commit all 8 dequant warps read it
//     back with tcgen05.ld, apply bias / activation / residual and store (or, with split-K,
//     atomically add) fp32.
// Every mbarrier wait is bounded; on expiry the CTA records error 3001, drains, releases its
// tensor memory and returns.
//
// Replaces the reference's q4k/q5k/q6k_gemm_ggml, tensor_core_q4k_gemm (WMMA), dp4a_q4k_gemm,
// dequant-to-f16/f32 + cuBLAS HGEMM/SGEMM and cuBLASLt FP8 call sites
// (src/cuda/executor/layers/cublas_prefill/gemm.rs:70-1100).
#include "common.cuh"
#include "tcgen05_common.cuh"
#include "../gemv_blocks.h"

namespace rlz {

__device__ int g_gemm_error = 0;

constexpr int GM_PRODUCERS = 256;      // dequant threads per 128-row tile (8 warps); the TMA warp and the MMA warp follow them
constexpr int GM_ROWS = 128;          // weight rows per CTA = MMA M
constexpr int GM_KSTEP = 64;          // K elements per stage (one 128-byte swizzle row of bf16)

struct GemmParams {
  const uint8_t* W; int64_t w_stride; int32_t qtype; int32_t n; int32_t k; int32_t m;
  const __nv_bfloat16* X; int64_t ldx;
  float* Y; int64_t ldy;
  const float* bias; const float* residual; int64_t ld_res;
  int32_t act; int32_t splitk; int32_t atomic_out; int32_t _pad;
  // tensor-parallel row-parallel GEMM: instead of storing, push {value, tag} pairs into this rank's slots of every
  // rank's inbox (peer memory); a reduce kernel on each rank sums the slots.  Layout of an inbox:
  // [2 alternating buffers][world * ar_splits writers][ar_rows token rows][ar_row_pairs] pairs; writer = rank * ar_splits
  // + K split; buffer = (epoch * ar_nsites + ar_site) & 1; tag = epoch * 256 + ar_site (epoch: device word, one per pass).
  uint2* ar_inbox[8];
  const uint32_t* ar_epoch;
  int64_t ar_row_pairs;
  int32_t ar_rank, ar_world, ar_rows, ar_enabled;
  int32_t ar_site, ar_nsites, ar_splits;
  int32_t flags;           // GM_OUT_BF16: Y is bf16 (ldy in elements); GM_RES_MUL: the `residual` operand multiplies instead of adding
  // ar_enabled == 2, two-shot all-reduce, first half (reduce-scatter by ownership): token row t belongs to rank t / rs_own_rows;
  // the CTA stores its fp32 tile (+ bias, + the local `residual` operand) only into the OWNER's inbox
  // [2 buffers][world writers][ar_splits][ar_rows owned rows][ar_row_pairs floats] (plain peer stores), then one thread fences
  // and publishes the tile's tag in the owner's flag array [2][world][ar_splits][rs_ntiles][rs_mtiles].  The owner's reduce
  // kernel (symm_mem.cu) sums the writers, normalises and sends finished rows to every rank.
  uint32_t* rs_flags[8];
  int32_t rs_own_rows, rs_ntiles, rs_mtiles, _pad2;
};
enum { GM_OUT_BF16 = 1, GM_RES_MUL = 2 };

// element i of an 8-entry array that lives in the kernel parameters, as a chain of selects: a run-time index would make the
// compiler copy the array to local memory
template <typename T>
__device__ __forceinline__ T pick8(T const (&a)[8], int i) {
  T v = a[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) v = i == j ? a[j] : v;
  return v;
}

// ---- producers: raw block bytes -> registers (issued one K step ahead), registers -> bf16 pairs -------------
// The integer code q of a weight is dropped into the mantissa of a bf16 power of two (magic + q is exact), the
// magic is subtracted again (exact) and one bf16x2 FMA applies scale and offset to two weights at a time:
//   PRMT (two code bytes -> two 16-bit lanes), LOP3 (mask | magic), HADD2, HFMA2  per pair.
// The scale (and the Q4_K / Q5_K minimum) is rounded to bf16 first; the operand fed to the tensor core is bf16 anyway.
struct RawW { uint4 r[5]; };

// bytes of one 256-weight block of a K-quant row in the device layout
template <int QT> struct BlockBytes { static constexpr int value = QT == QT_Q4_K ? 144 : QT == QT_Q5_K ? 176 : QT == QT_Q6_K ? Q6K_DEV_STRIDE : 0; };

// the bytes of one thread's 32 weights of K group g (0..3) of the block at `blk` (global or shared memory)
template <int QT>
__device__ __forceinline__ void load_block(const uint8_t* blk, int g, int half, RawW& w) {
  if (QT == QT_Q4_K || QT == QT_Q5_K) {
    w.r[0] = *(const uint4*)blk;
    const uint8_t* qs = blk + (QT == QT_Q5_K ? 48 : 16) + 32 * g;
    w.r[1] = *(const uint4*)qs; w.r[2] = *(const uint4*)(qs + 16);
    if (QT == QT_Q5_K) { w.r[3] = *(const uint4*)(blk + 16); w.r[4] = *(const uint4*)(blk + 32); }
  } else if (QT == QT_Q6_K) {
    const int n = g >> 1, upper = g & 1;
    const uint8_t* ql = blk + 64 * n + 32 * half;
    const uint8_t* qh = blk + 128 + 32 * n;
    w.r[0] = *(const uint4*)ql; w.r[1] = *(const uint4*)(ql + 16);
    w.r[2] = *(const uint4*)qh; w.r[3] = *(const uint4*)(qh + 16);
    w.r[4].x = *(const uint32_t*)(blk + 192 + 8 * n + 4 * upper);     // the four int8 scales of this 64-column group
    w.r[4].y = *(const uint32_t*)(blk + 208);                          // d (f16) in the low half
  }
}

template <int QT> struct IsLegacy { static constexpr bool value = QT == QT_Q4_0 || QT == QT_Q4_1 || QT == QT_Q5_0 || QT == QT_Q5_1 || QT == QT_Q8_0; };

// 32-weight block types: one thread's half of a 64-column K step is exactly one block.  r[0] (and r[1] for Q8_0) = the code
// bytes, r[2].x = d (and m) as two fp16, r[2].y = the 32 fifth bits.  Q4_0 / Q8_0 rows are planar on the device (all block
// scales first, then the codes, both 16-byte aligned); the others keep their stored interleaved blocks, whose code bytes are
// only 2- or 4-byte aligned.
template <int QT>
__device__ __forceinline__ void load_legacy(const uint8_t* row, int k, int k0, int half, RawW& w) {
  const int b = (k0 >> 5) + half;
  if (QT == QT_Q4_0 || QT == QT_Q8_0) {
    const uint8_t* qs = row + dev_planar_qoff(k >> 5);
    w.r[2].x = *(const uint16_t*)(row + 2 * b);
    if (QT == QT_Q4_0) w.r[0] = __ldg((const uint4*)(qs + 16 * b));
    else { w.r[0] = __ldg((const uint4*)(qs + 32 * b)); w.r[1] = __ldg((const uint4*)(qs + 32 * b + 16)); }
  } else if (QT == QT_Q4_1) {
    const uint32_t* blk = (const uint32_t*)(row + 20 * b);
    w.r[2].x = blk[0];
    w.r[0] = make_uint4(blk[1], blk[2], blk[3], blk[4]);
  } else if (QT == QT_Q5_1) {
    const uint32_t* blk = (const uint32_t*)(row + 24 * b);
    w.r[2].x = blk[0]; w.r[2].y = blk[1];
    w.r[0] = make_uint4(blk[2], blk[3], blk[4], blk[5]);
  } else {                                                                  // Q5_0: 22-byte blocks, 2-byte aligned
    const uint16_t* blk = (const uint16_t*)(row + 22 * b);
    w.r[2].x = blk[0];
    w.r[2].y = (uint32_t)blk[1] | ((uint32_t)blk[2] << 16);
    w.r[0] = make_uint4((uint32_t)blk[3] | ((uint32_t)blk[4] << 16), (uint32_t)blk[5] | ((uint32_t)blk[6] << 16),
                        (uint32_t)blk[7] | ((uint32_t)blk[8] << 16), (uint32_t)blk[9] | ((uint32_t)blk[10] << 16));
  }
}

template <int QT>
__device__ __forceinline__ void load_raw(const uint8_t* row, int k, int k0, int half, RawW& w) {
  const int sb = k0 >> 8, g = (k0 >> 6) & 3;
  if (QT == QT_Q4_K || QT == QT_Q5_K || QT == QT_Q6_K) {
    load_block<QT>(row + (int64_t)sb * BlockBytes<QT>::value, g, half, w);
  } else if (IsLegacy<QT>::value) {
    load_legacy<QT>(row, k, k0, half, w);
  } else {                                                                  // BF16 / F16: 32 elements = 64 bytes
    const uint4* src = (const uint4*)(row + (int64_t)(k0 + 32 * half) * 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) w.r[i] = __ldg(src + i);
  }
}

__device__ __forceinline__ uint32_t bf2_splat(float x) { const __nv_bfloat162 v = __float2bfloat162_rn(x); return *(const uint32_t*)&v; }
__device__ __forceinline__ float bf_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// (codes | magic) - magic, then * scale + offset, two weights per call; all operands packed bf16x2
__device__ __forceinline__ uint32_t bf2_affine(uint32_t codes_magic, uint32_t magic, uint32_t scale, uint32_t offset) {
  const __nv_bfloat162 q = __hsub2(*(const __nv_bfloat162*)&codes_magic, *(const __nv_bfloat162*)&magic);
  const __nv_bfloat162 v = __hfma2(q, *(const __nv_bfloat162*)&scale, *(const __nv_bfloat162*)&offset);
  return *(const uint32_t*)&v;
}

template <int QT>
__device__ __forceinline__ void dequant_raw32(const RawW& w, int k0, int half, uint32_t* out) {
  const int g = (k0 >> 6) & 3;
  if (QT == QT_Q4_K || QT == QT_Q5_K) {
    constexpr bool q5 = QT == QT_Q5_K;
    const uint4 hdr = w.r[0];
    const float d = h2f_alu(hdr.x & 0xFFFFu), dmin = h2f_alu(hdr.x >> 16);
    const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
    const uint32_t sc2 = bf2_splat(d * (float)k4_pick(ks.sc_lo, ks.sc_hi, 2 * g + half));
    const uint32_t mn2 = bf2_splat(-dmin * (float)k4_pick(ks.m_lo, ks.m_hi, 2 * g + half));
    // codes sit at bits 3..6 (Q4_K: magic 16, ulp 1/8) or 2..6 (Q5_K: magic 32, ulp 1/4) of their byte
    constexpr uint32_t MAGIC = q5 ? 0x42004200u : 0x41804180u;
    const uint32_t qw[8] = {w.r[1].x, w.r[1].y, w.r[1].z, w.r[1].w, w.r[2].x, w.r[2].y, w.r[2].z, w.r[2].w};
    const uint32_t hw[8] = {w.r[3].x, w.r[3].y, w.r[3].z, w.r[3].w, w.r[4].x, w.r[4].y, w.r[4].z, w.r[4].w};
    const int hsh = 2 * g + half;
#pragma unroll
    for (int i = 0; i < 8; ++i) {                         // word i holds elements 4i..4i+3 of this half
      uint32_t ws;
      if (q5) ws = ((half ? qw[i] >> 2 : qw[i] << 2) & 0x3C3C3C3Cu) | (((hw[i] >> hsh) << 6) & 0x40404040u);
      else ws = (half ? qw[i] >> 1 : qw[i] << 3) & 0x78787878u;
      out[2 * i] = bf2_affine(__byte_perm(ws, 0, 0x4140) | MAGIC, MAGIC, sc2, mn2);
      out[2 * i + 1] = bf2_affine(__byte_perm(ws, 0, 0x4342) | MAGIC, MAGIC, sc2, mn2);
    }
  } else if (QT == QT_Q6_K) {
    const int upper = g & 1, part = half;
    const float d = h2f_alu(w.r[4].y & 0xFFFFu);
    const uint32_t scw = w.r[4].x;
    const int s0i = (int)(int8_t)((scw >> (16 * part)) & 0xFFu), s1i = (int)(int8_t)((scw >> (16 * part + 8)) & 0xFFu);
    const uint32_t s0 = bf2_splat(d * (float)s0i), s1 = bf2_splat(d * (float)s1i);
    constexpr uint32_t MAGIC = 0x42804280u;               // 64: codes at bits 1..6 of their byte (ulp 1/2)
    constexpr uint32_t MAGIC_OFF = 0x42C042C0u;           // 96 = 64 + 32: subtracting it also centres the code (q - 32)
    const uint32_t lq[8] = {w.r[0].x, w.r[0].y, w.r[0].z, w.r[0].w, w.r[1].x, w.r[1].y, w.r[1].z, w.r[1].w};
    const uint32_t hq[8] = {w.r[2].x, w.r[2].y, w.r[2].z, w.r[2].w, w.r[3].x, w.r[3].y, w.r[3].z, w.r[3].w};
    const int hs = 2 * (2 * upper + part);
#pragma unroll
    for (int w4 = 0; w4 < 8; ++w4) {
      const uint32_t ws = ((upper ? lq[w4] >> 3 : lq[w4] << 1) & 0x1E1E1E1Eu) | (((hq[w4] >> hs) << 5) & 0x60606060u);
      const uint32_t s = w4 < 4 ? s0 : s1;
      out[2 * w4] = bf2_affine(__byte_perm(ws, 0, 0x4140) | MAGIC, MAGIC_OFF, s, 0u);
      out[2 * w4 + 1] = bf2_affine(__byte_perm(ws, 0, 0x4342) | MAGIC, MAGIC_OFF, s, 0u);
    }
  } else if (IsLegacy<QT>::value) {
    // element e < 16 is the low nibble of code byte e, element 16 + e its high nibble (Q8_0: byte e is element e);
    // value = d * (q - 8 | q - 16 | q) or d * q + m
    const float d = h2f_alu(w.r[2].x & 0xFFFFu);
    const float m = (QT == QT_Q4_1 || QT == QT_Q5_1) ? h2f_alu(w.r[2].x >> 16) : QT == QT_Q4_0 ? -8.f * d : QT == QT_Q5_0 ? -16.f * d : 0.f;
    if (QT == QT_Q8_0) {
      const uint32_t q[8] = {w.r[0].x, w.r[0].y, w.r[0].z, w.r[0].w, w.r[1].x, w.r[1].y, w.r[1].z, w.r[1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a = (float)(int8_t)(q[i] & 0xFFu), b = (float)(int8_t)((q[i] >> 8) & 0xFFu);
        const float c = (float)(int8_t)((q[i] >> 16) & 0xFFu), e = (float)(int8_t)(q[i] >> 24);
        out[2 * i] = pack_bf16(d * a, d * b);
        out[2 * i + 1] = pack_bf16(d * c, d * e);
      }
    } else {
      const uint32_t q[4] = {w.r[0].x, w.r[0].y, w.r[0].z, w.r[0].w};
      const uint32_t qh = w.r[2].y;
      constexpr bool five = QT == QT_Q5_0 || QT == QT_Q5_1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {                        // word i: code bytes 4i .. 4i+3
        float lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t byte = (q[i] >> (8 * j)) & 0xFFu;
          uint32_t l = byte & 15u, h = byte >> 4;
          if (five) { l |= ((qh >> (4 * i + j)) & 1u) << 4; h |= ((qh >> (16 + 4 * i + j)) & 1u) << 4; }
          lo[j] = fmaf(d, (float)l, m); hi[j] = fmaf(d, (float)h, m);
        }
        out[2 * i] = pack_bf16(lo[0], lo[1]); out[2 * i + 1] = pack_bf16(lo[2], lo[3]);
        out[8 + 2 * i] = pack_bf16(hi[0], hi[1]); out[8 + 2 * i + 1] = pack_bf16(hi[2], hi[3]);
      }
    }
  } else if (QT == QT_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { out[4 * i] = w.r[i].x; out[4 * i + 1] = w.r[i].y; out[4 * i + 2] = w.r[i].z; out[4 * i + 3] = w.r[i].w; }
  } else {                                                // F16
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t x[4] = {w.r[i].x, w.r[i].y, w.r[i].z, w.r[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) out[4 * i + j] = pack_bf16(h2f_alu(x[j] & 0xFFFFu), h2f_alu(x[j] >> 16));
    }
  }
}

// store 32 bf16 (16 words) as columns [32*half, 32*half+32) of row r of a [rows x 64] K-major SWIZZLE_128B tile
__device__ __forceinline__ void store_half_row_sw128(uint8_t* tile, int r, int half, const uint32_t* v) {
  uint8_t* base = tile + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = 4 * half + j;
    *(uint4*)(base + ((c ^ (r & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
}

// RT = 128-row weight tiles per CTA (1 or 2).  With RT = 2 the CTA owns 256 weight rows, keeps two accumulators in TMEM
// and issues two MMAs per K slice that share the activation tile, which halves the activation traffic from L2 per FLOP.
// Optional phase trace (diagnostics): thread 0 of each of the first GM_TRACE_CTAS CTAs records the global timer at fixed points.
constexpr int GM_TRACE_CTAS = 1024, GM_TRACE_PTS = 8;
__device__ int g_gemm_trace_on = 0;
__device__ unsigned long long g_gemm_trace[GM_TRACE_CTAS * GM_TRACE_PTS];
__device__ __forceinline__ void gm_trace(bool on, int cta, int pt) {
  if (on) {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_gemm_trace[cta * GM_TRACE_PTS + pt] = t;
  }
}

// K-quant weights do not go through the load/store units at all: a third single-thread role streams the raw 256-weight
// blocks of the CTA's rows with TMA (box = rows x block bytes) into a two-deep shared-memory ring, one block per four K steps,
// and the dequant warps read their row's bytes from there.  Row-strided 16-byte global loads (one sector per lane) were the
// limit of the earlier version (lg_throttle / long_scoreboard).  Dense bf16 / f16 weights keep the register prefetch ring.
template <int NT, int QT, int RT> struct GemmCfg {
  static constexpr bool RAWTMA = QT == QT_Q4_K || QT == QT_Q5_K || QT == QT_Q6_K;
  static constexpr int ROWS = RT * GM_ROWS;
  // token tiles <= 64 (decode batches, K split across CTAs): shared memory is kept under half an SM so that two CTAs are
  // resident and the split-K grid runs as one wave; the ring is shallow because the dequant warps, not the MMAs, set the pace
  static constexpr int STAGES = RAWTMA ? (RT == 2 ? 2 : NT == 256 ? 3 : NT <= 64 ? (BlockBytes<QT>::value <= 144 ? 3 : 2) : 4) : (RT == 2 ? 3 : 4);
  static constexpr int RAW_BYTES = RAWTMA ? ROWS * BlockBytes<QT>::value : 0;      // one ring slot
  static constexpr int STAGE = ROWS * 128 + NT * 128;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE + 2 * RAW_BYTES + 1024;
  static_assert(NT > 64 || !RAWTMA || 2 * SMEM <= 226 * 1024, "decode-size tiles must fit twice per SM");
  static constexpr int THREADS = RT * GM_PRODUCERS + 96;                           // dequant warps + B TMA + MMA + raw TMA
};

// RS: the reduce-scatter epilogue of the two-shot all-reduce is compiled in (its own instantiations, so that the register
// allocation of every other launch stays what it was).
template <int NT, int QT, int RT, bool RS>
__global__ void __launch_bounds__(RT * GM_PRODUCERS + 96) gemm_kquant_tcgen05_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                                                     const __grid_constant__ CUtensorMap wmap) {
  using Cfg = GemmCfg<NT, QT, RT>;
  constexpr int GM_STAGES = Cfg::STAGES;
  constexpr bool RAWTMA = Cfg::RAWTMA;
  constexpr int PRODUCERS = RT * GM_PRODUCERS, PWARPS = PRODUCERS / 32, ROWS = RT * GM_ROWS;
  extern __shared__ __align__(1024) uint8_t gsm[];
  __shared__ __align__(8) uint64_t full_bar[GM_STAGES], empty_bar[GM_STAGES], done_bar, raw_full[2], raw_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * ROWS, m0 = blockIdx.y * NT;
  const int cta_lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  const bool tr = tid == 0 && cta_lin < GM_TRACE_CTAS && g_gemm_trace_on;
  gm_trace(tr, cta_lin, 0);
  uint8_t* sm = (uint8_t*)(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = ROWS * 128, B_BYTES = NT * 128, STAGE = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = RT * NT < 32 ? 32 : RT * NT;

  if (tid == 0) {
    failed_s = 0;
    for (int s = 0; s < GM_STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gm_smem_u32(&full_bar[s])), "r"(PWARPS + 1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&empty_bar[s])));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&done_bar)));
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&raw_full[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gm_smem_u32(&raw_empty[i])), "r"(PWARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {                                        // one warp allocates the accumulator columns of tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_s;
  gm_trace(tr, cta_lin, 1);
  pdl_launch_dependents();
  pdl_wait();
  gm_trace(tr, cta_lin, 2);

  // K range of this split
  const int ksteps_total = p.k / GM_KSTEP;
  const int per = (ksteps_total + p.splitk - 1) / p.splitk;
  const int ks0 = blockIdx.z * per, ks1 = min(ksteps_total, ks0 + per);
  const int nit = max(0, ks1 - ks0);
  bool ok = true;

  if (warp < PWARPS) {
    // ---- dequant producers: thread -> (row, half of the 64-column step) ---------------------
    const int r = tid & (ROWS - 1), half = tid / ROWS;
    const int wrow = n0 + r;
    const uint8_t* wptr = p.W + (int64_t)min(wrow, p.n - 1) * p.w_stride;
    if constexpr (RAWTMA) {
      constexpr int BB = BlockBytes<QT>::value;
      const uint8_t* raw = sm + GM_STAGES * STAGE;          // ring of two block tiles [ROWS][BB]; rows past n arrive zero-filled
      const int kb0 = ks0 >> 2;
      for (int it = 0; it < nit; ++it) {
        const int step = ks0 + it, kbi = (step >> 2) - kb0, g = step & 3, rb = kbi & 1, s = it % GM_STAGES;
        if (it == 0 || g == 0) {                            // first step of a block: its bytes have landed
          ok = gm_wait(&raw_full[rb], (uint32_t)(kbi >> 1) & 1u);
          if (!ok) break;
          if (it == 0) gm_trace(tr, cta_lin, 3);
        }
        if (it >= GM_STAGES) {                              // the MMAs that read this stage GM_STAGES steps ago are done
          ok = gm_wait(&empty_bar[s], (uint32_t)(it / GM_STAGES - 1) & 1u);
          if (!ok) break;
        }
        RawW w;
        load_block<QT>(raw + (size_t)rb * Cfg::RAW_BYTES + (size_t)r * BB, g, half, w);
        uint32_t v[16];
        dequant_raw32<QT>(w, step * GM_KSTEP, half, v);
        store_half_row_sw128(sm + s * STAGE, r, half, v);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) {
          gm_arrive(&full_bar[s]);
          if (g == 3 || it == nit - 1) gm_arrive(&raw_empty[rb]);       // this warp is done with the block tile
        }
      }
    } else {
    // a ring of PF K steps of raw block bytes per thread keeps enough loads in flight to cover HBM latency
    constexpr int PF = NT <= 64 ? 2 : RT == 2 ? (QT == QT_Q4_K ? 3 : 2) : (QT == QT_Q4_K ? 4 : 3);   // short kernels: smaller code wins
    RawW ring[PF];
#pragma unroll
    for (int j = 0; j < PF; ++j)
      if (j < nit) load_raw<QT>(wptr, p.k, (ks0 + j) * GM_KSTEP, half, ring[j]);
    for (int it0 = 0; it0 < nit && ok; it0 += PF) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int it = it0 + j;
        if (it >= nit) break;
        const int s = it % GM_STAGES;
        if (it >= GM_STAGES) {                            // the MMAs that read this stage GM_STAGES steps ago are done
          ok = gm_wait(&empty_bar[s], (uint32_t)(it / GM_STAGES - 1) & 1u);
          if (!ok) break;
        }
        uint32_t v[16];
        if (wrow < p.n) dequant_raw32<QT>(ring[j], (ks0 + it) * GM_KSTEP, half, v);
        else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0u;
        }
        if (it + PF < nit) load_raw<QT>(wptr, p.k, (ks0 + it + PF) * GM_KSTEP, half, ring[j]);   // refill the slot just consumed
        store_half_row_sw128(sm + s * STAGE, r, half, v);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) gm_arrive(&full_bar[s]);
      }
    }
    }
  } else if (warp == PWARPS + 2) {
    // ---- raw weight blocks by TMA (K-quants): one [ROWS x block] tile per four K steps, two in flight ----
    if (RAWTMA && lane == 0) {
      constexpr int BB = BlockBytes<QT>::value;
      uint8_t* raw = sm + GM_STAGES * STAGE;
      const int kb0 = ks0 >> 2, nkb = nit > 0 ? ((ks1 - 1) >> 2) - kb0 + 1 : 0;
      for (int kbi = 0; kbi < nkb; ++kbi) {
        const int rb = kbi & 1;
        if (kbi >= 2) {                                     // every dequant warp has finished with the tile two blocks ago
          ok = gm_wait(&raw_empty[rb], (uint32_t)((kbi >> 1) - 1) & 1u);
          if (!ok) break;
        }
        gm_arrive_expect_tx(&raw_full[rb], (uint32_t)Cfg::RAW_BYTES);
        tma_load_2d(raw + (size_t)rb * Cfg::RAW_BYTES, &wmap, (kb0 + kbi) * BB, n0, &raw_full[rb]);
      }
    }
  } else if (warp == PWARPS) {
    // ---- TMA producer: activations of this token tile -------------------------------------------
    if (lane == 0) {
      for (int it = 0; it < nit; ++it) {
        const int s = it % GM_STAGES;
        if (it >= GM_STAGES) {
          ok = gm_wait(&empty_bar[s], (uint32_t)(it / GM_STAGES - 1) & 1u);
          if (!ok) break;
        }
        uint8_t* Bt = sm + s * STAGE + A_BYTES;
        gm_arrive_expect_tx(&full_bar[s], (uint32_t)B_BYTES);
        tma_load_2d(Bt, &xmap, (ks0 + it) * GM_KSTEP, m0, &full_bar[s]);
      }
    }
  } else if (warp == PWARPS + 1) {
    // ---- MMA issuer --------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(GM_ROWS, NT);
      for (int it = 0; it < nit; ++it) {
        const int s = it % GM_STAGES;
        ok = gm_wait(&full_bar[s], (uint32_t)(it / GM_STAGES) & 1u);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t db = make_sdesc_k_sw128(gm_smem_u32(sm + s * STAGE + A_BYTES));
#pragma unroll
        for (int kk = 0; kk < GM_KSTEP / 16; ++kk) {      // advance 32 bytes (two 16-byte units) per K=16 slice
#pragma unroll
          for (int j = 0; j < RT; ++j) {                  // row tile j: rows 128j.. of the A stage, accumulator columns NT*j..
            const uint64_t da = make_sdesc_k_sw128(gm_smem_u32(sm + s * STAGE + j * GM_ROWS * 128));
            umma_bf16(tmem_d + (uint32_t)(j * NT), da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), idesc, (it > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&done_bar);                     // arrives when every MMA above has completed
    }
  }
  if (!ok) { failed_s = 1; atomicExch(&g_gemm_error, 3001); }
  gm_trace(tr, cta_lin, 4);

  // ---- epilogue: TMEM lane = weight row, column = token; each warp a lane quarter x column half (x row tile) ----
  // (a K split without work still pushes zeros in all-reduce mode: the reducer counts on every writer)
  if (warp < PWARPS && (nit > 0 || p.ar_enabled)) {
    if (ok && nit > 0 && !gm_wait(&done_bar, 0u)) { ok = false; failed_s = 1; atomicExch(&g_gemm_error, 3001); }
    gm_trace(tr, cta_lin, 5);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    constexpr int COLS_PER_WARP = NT >= 64 ? NT / 2 : NT;
    const int q = warp & 3, chalf = (warp >> 2) & 1, rt = warp >> 3;
    if (ok && (NT >= 64 || chalf == 0)) {
      const int row = n0 + rt * GM_ROWS + q * 32 + lane;
      const float bias = (p.bias && row < p.n && blockIdx.z == 0) ? p.bias[row] : 0.f;
      const uint32_t epoch = p.ar_enabled ? *p.ar_epoch : 0u;
      const uint32_t tag = epoch * 256u + (uint32_t)p.ar_site;
      const int64_t ar_buf = (int64_t)((epoch * (uint32_t)p.ar_nsites + (uint32_t)p.ar_site) & 1u) * p.ar_world * p.ar_splits;
      const int64_t ar_slot = (ar_buf + (int64_t)p.ar_rank * p.ar_splits + blockIdx.z) * p.ar_rows * p.ar_row_pairs;
#pragma unroll 1
      for (int c0 = chalf * COLS_PER_WARP; c0 < (chalf + 1) * COLS_PER_WARP; c0 += 32) {
        if (m0 + c0 >= p.m) break;                        // warp-uniform: no tokens left in this tile
        uint32_t r[32];
        const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(rt * NT + c0);
        if (nit == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        } else
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
              "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
              "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.n) {
          // one compact loop per output mode (the mode is uniform over the launch): only the code of the mode in use is fetched
          const int ntok = min(32, p.m - (m0 + c0));
          float* dst = p.Y + (int64_t)(m0 + c0) * p.ldy + row;
          if (RS && p.ar_enabled == 2) {                  // reduce-scatter: each token row goes to its owner only (4-byte stores, lanes = consecutive features)
            const float* res = (p.residual && blockIdx.z == 0) ? p.residual + (int64_t)(m0 + c0) * p.ld_res + row : nullptr;
            const int64_t slot_row0 = (ar_buf + (int64_t)p.ar_rank * p.ar_splits + blockIdx.z) * p.ar_rows;
            int owner = (m0 + c0) / p.rs_own_rows, lt = (m0 + c0) - owner * p.rs_own_rows;      // advanced incrementally: no division per token
            float* dst_o = (float*)pick8(p.ar_inbox, owner) + (slot_row0 + lt) * p.ar_row_pairs + row;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < ntok) {
                float v = __uint_as_float(r[j]) + bias;
                if (res) v += res[(int64_t)j * p.ld_res];
                *dst_o = v;
                dst_o += p.ar_row_pairs;
                if (++lt == p.rs_own_rows) { lt = 0; ++owner; dst_o = (float*)pick8(p.ar_inbox, owner) + slot_row0 * p.ar_row_pairs + row; }
              }
            }
          } else if (p.ar_enabled) {                      // one 8-byte store per rank; lanes cover consecutive rows (coalesced)
            const int64_t off0 = ar_slot + (int64_t)(m0 + c0) * p.ar_row_pairs + row;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ntok)
                for (int pr = 0; pr < p.ar_world; ++pr) st_pair_sys(p.ar_inbox[pr] + off0 + (int64_t)j * p.ar_row_pairs, __float_as_uint(__uint_as_float(r[j]) + bias), tag);
          } else if (p.atomic_out) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ntok) atomicAdd(dst + (int64_t)j * p.ldy, __uint_as_float(r[j]) + bias);
          } else if (p.act == ACT_NONE && !p.residual && !p.flags) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ntok) dst[(int64_t)j * p.ldy] = __uint_as_float(r[j]) + bias;
          } else {
            const float* res = p.residual ? p.residual + (int64_t)(m0 + c0) * p.ld_res + row : nullptr;
            const bool mul = (p.flags & GM_RES_MUL) != 0, to_bf16 = (p.flags & GM_OUT_BF16) != 0;
            __nv_bfloat16* dst16 = (__nv_bfloat16*)p.Y + (int64_t)(m0 + c0) * p.ldy + row;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < ntok) {
                float v = __uint_as_float(r[j]) + bias;
                if (p.act == ACT_GELU) v = gelu_tanh(v); else if (p.act == ACT_SILU) v = silu(v);
                if (res) v = mul ? v * res[(int64_t)j * p.ld_res] : v + res[(int64_t)j * p.ld_res];
                if (to_bf16) dst16[(int64_t)j * p.ldy] = __float2bfloat16_rn(v);      // the operand of the next GEMM, written where it is read
                else dst[(int64_t)j * p.ldy] = v;
              }
            }
          }
        }
      }
    }
  }
  gm_trace(tr, cta_lin, 6);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (RS && p.ar_enabled == 2 && tid == 0 && !failed_s) {
    // every epilogue thread's peer stores happened before the barrier; the fence makes them visible system-wide before the flag
    __threadfence_system();
    const uint32_t epoch = *p.ar_epoch;
    const uint32_t tag = epoch * 256u + (uint32_t)p.ar_site;
    const int64_t par = (int64_t)((epoch * (uint32_t)p.ar_nsites + (uint32_t)p.ar_site) & 1u);
    const int64_t fidx = (((par * p.ar_world + p.ar_rank) * p.ar_splits + blockIdx.z) * p.rs_ntiles + blockIdx.x) * p.rs_mtiles + blockIdx.y;
    const int mend = min(p.m, m0 + NT);
    for (int owner = m0 / p.rs_own_rows; owner <= (mend - 1) / p.rs_own_rows; ++owner)
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(pick8(p.rs_flags, owner) + fidx), "r"(tag) : "memory");
  }
  if (failed_s && warp == PWARPS && lane == 0) {
    // error path: give TMA copies still in flight a bounded chance to land before the CTA's shared memory is released
    for (int s = 0; s < GM_STAGES && s < nit; ++s) gm_wait(&full_bar[s], 0u);
    if (RAWTMA && nit > 0) gm_wait(&raw_full[0], 0u);
  }
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
}

// ---- host side: tensor map for the activations, launch --------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// X viewed as a 2-D bf16 tensor [m rows, k columns] with a row pitch of ldx elements; boxes of [box_rows x 64]
static int make_x_map(CUtensorMap* map, const GemmParams& p, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return -6;
  const cuuint64_t gdim[2] = {(cuuint64_t)p.k, (cuuint64_t)p.m};
  const cuuint64_t gstride[1] = {(cuuint64_t)p.ldx * 2};
  const cuuint32_t box[2] = {(cuuint32_t)GM_KSTEP, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)p.X, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -7;
}

// W viewed as a 2-D byte tensor [n rows, row bytes] with a row pitch of w_stride; boxes of [box_rows x block bytes]
static int make_w_map(CUtensorMap* map, const GemmParams& p, int box_rows, int block_bytes) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return -6;
  const cuuint64_t gdim[2] = {(cuuint64_t)(p.k / 256) * block_bytes, (cuuint64_t)p.n};
  const cuuint64_t gstride[1] = {(cuuint64_t)p.w_stride};
  const cuuint32_t box[2] = {(cuuint32_t)block_bytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)p.W, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -7;
}

template <int NT, int QT, int RT, bool RS>
int launch_gemm_rs(const GemmParams& p, cudaStream_t st) {
  using Cfg = GemmCfg<NT, QT, RT>;
  const size_t smem = Cfg::SMEM;
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(gemm_kquant_tcgen05_kernel<NT, QT, RT, RS>, smem, 0); e != cudaSuccess) return (int)e;
  alignas(64) CUtensorMap xmap, wmap;
  int rc = make_x_map(&xmap, p, NT);
  if (rc) return rc;
  if (Cfg::RAWTMA) rc = make_w_map(&wmap, p, Cfg::ROWS, BlockBytes<QT>::value);
  else wmap = xmap;                                        // unused by the dense-weight instantiations
  if (rc) return rc;
  dim3 grid((p.n + RT * GM_ROWS - 1) / (RT * GM_ROWS), (p.m + NT - 1) / NT, p.splitk);
  return (int)launch(gemm_kquant_tcgen05_kernel<NT, QT, RT, RS>, grid, dim3(Cfg::THREADS), smem, st, p, xmap, wmap);
}
template <int NT, int QT, int RT>
int launch_gemm_q(const GemmParams& p, cudaStream_t st) {
  return p.ar_enabled == 2 ? launch_gemm_rs<NT, QT, RT, true>(p, st) : launch_gemm_rs<NT, QT, RT, false>(p, st);
}

template <int NT, int RT>
int launch_gemm(const GemmParams& p, cudaStream_t st) {
  switch (p.qtype) {
    case QT_Q4_K: return launch_gemm_q<NT, QT_Q4_K, RT>(p, st);
    case QT_Q5_K: return launch_gemm_q<NT, QT_Q5_K, RT>(p, st);
    case QT_Q6_K: return launch_gemm_q<NT, QT_Q6_K, RT>(p, st);
    case QT_BF16: return launch_gemm_q<NT, QT_BF16, RT>(p, st);
    case QT_F16: return launch_gemm_q<NT, QT_F16, RT>(p, st);
    default: break;
  }
  if constexpr (RT == 1) {                                 // the 32-weight block types run 128-row CTAs only
    switch (p.qtype) {
      case QT_Q4_0: return launch_gemm_q<NT, QT_Q4_0, 1>(p, st);
      case QT_Q4_1: return launch_gemm_q<NT, QT_Q4_1, 1>(p, st);
      case QT_Q5_0: return launch_gemm_q<NT, QT_Q5_0, 1>(p, st);
      case QT_Q5_1: return launch_gemm_q<NT, QT_Q5_1, 1>(p, st);
      case QT_Q8_0: return launch_gemm_q<NT, QT_Q8_0, 1>(p, st);
      default: break;
    }
  }
  return -2;
}

}  // namespace rlz

extern "C" {

// 0 / error code recorded by a GEMM CTA whose bounded mbarrier wait expired (3001)
int rlz_gemm_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, rlz::g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) { int z = 0; cudaMemcpyToSymbol(rlz::g_gemm_error, &z, sizeof(int)); }
  return v;
}

// Tile shape the launcher picks for a call: tokens per CTA, weight rows per CTA, K splits (after clamping).  The owner-side
// reduce kernel of the two-shot all-reduce needs them to know which tile flags cover a token row.
int rlz_gemm_plan(const rlz::GemmParams* pp, int* nt, int* rows, int* splitk) {
  using namespace rlz;
  const GemmParams& p = *pp;
  if (p.k % GM_KSTEP || p.m < 1 || p.n < 1) return -1;
  int sk = p.splitk < 1 ? 1 : p.splitk;
  if (sk > p.k / GM_KSTEP) sk = p.k / GM_KSTEP;
  if (p.ar_enabled == 1) sk = p.ar_splits;
  *splitk = sk;
  *rows = GM_ROWS;
  if (p.m <= 32) { *nt = 32; return 0; }
  if (p.m <= 64) { *nt = 64; return 0; }
  if (p.m <= 128) { *nt = 128; return 0; }
  *nt = 256;
  const long long tiles1 = (long long)((p.n + 127) / 128) * ((p.m + 255) / 256) * sk;
  const long long tiles2 = (long long)((p.n + 255) / 256) * ((p.m + 255) / 256) * sk;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool legacy = p.qtype == QT_Q4_0 || p.qtype == QT_Q4_1 || p.qtype == QT_Q5_0 || p.qtype == QT_Q5_1 || p.qtype == QT_Q8_0;
  const bool wide_fits = !(p.qtype == QT_Q5_K || p.qtype == QT_Q6_K || legacy);
  const long long cost1 = ((tiles1 + sms - 1) / sms) * 840, cost2 = ((tiles2 + sms - 1) / sms) * 1100;
  if (wide_fits && (p._pad == 2 || (p._pad != 1 && cost2 < cost1))) *rows = 2 * GM_ROWS;
  return 0;
}

// Y[m, n] = act(X[m, k] W^T + bias) + residual.  With splitk > 1 the partial products are added
// atomically into Y, which the caller must have initialised (zeros, or the residual); bias is added
// by split 0 and no activation is applied.  Returns 0, a negative code for bad arguments or a cudaError_t.
int rlz_gemm_kquant(const rlz::GemmParams* pp, void* stream) {
  using namespace rlz;
  GemmParams p = *pp;
  if (p.k % GM_KSTEP || p.m < 1 || p.n < 1) return -1;
  const bool legacy = p.qtype == QT_Q4_0 || p.qtype == QT_Q4_1 || p.qtype == QT_Q5_0 || p.qtype == QT_Q5_1 || p.qtype == QT_Q8_0;
  if (!(p.qtype == QT_Q4_K || p.qtype == QT_Q5_K || p.qtype == QT_Q6_K || p.qtype == QT_BF16 || p.qtype == QT_F16 || legacy)) return -2;
  if ((p.qtype == QT_Q4_K || p.qtype == QT_Q5_K || p.qtype == QT_Q6_K) && p.k % 256) return -3;
  if (((uintptr_t)p.X & 15) || (p.ldx % 8) || ((uintptr_t)p.W & 15) || (p.w_stride & 15)) return -4;
  if (p.splitk < 1) p.splitk = 1;
  if (p.splitk > p.k / GM_KSTEP) p.splitk = p.k / GM_KSTEP;
  p.atomic_out = (p.splitk > 1 && !p.ar_enabled) ? 1 : 0;
  if (p.atomic_out && (p.act != ACT_NONE || p.flags)) return -5;
  if (p.ar_enabled && p.flags) return -8;
  if (p.ar_enabled == 2) {
    if (p.splitk > p.ar_splits || p.act != ACT_NONE || p.ar_world < 1 || p.ar_world > 8 || p.rs_own_rows < 1 || p.rs_own_rows > p.ar_rows ||
        (long long)p.rs_own_rows * p.ar_world < p.m || p.n > p.ar_row_pairs || p.ar_site < 0 || p.ar_site >= 256 || p.ar_site >= p.ar_nsites ||
        (p.n + GM_ROWS - 1) / GM_ROWS > p.rs_ntiles || (p.m + 31) / 32 > p.rs_mtiles) return -8;
  } else if (p.ar_enabled) {
    if (p.splitk > p.ar_splits || p.act != ACT_NONE || p.residual || p.ar_world < 1 || p.ar_world > 8 || p.m > p.ar_rows ||
        p.n > p.ar_row_pairs || p.ar_site < 0 || p.ar_site >= 256 || p.ar_site >= p.ar_nsites) return -8;
    p.splitk = p.ar_splits;                               // the reducer expects exactly ar_splits writers per rank
  }
  if ((p.ldx * 2) % 16) return -4;
  cudaStream_t st = (cudaStream_t)stream;
  if (p.m <= 32) return launch_gemm<32, 1>(p, st);
  if (p.m <= 64) return launch_gemm<64, 1>(p, st);
  if (p.m <= 128) return launch_gemm<128, 1>(p, st);
  // 128- or 256-row CTAs: whichever needs less time by a two-term model - waves of CTAs over the SMs times the measured cost
  // of one K step of a CTA (128 rows: ~840 cycles, set by its 8 dequant warps; 256 rows: ~1100 cycles, set by the MMAs).
  // p._pad forces the choice (1 = 128 rows, 2 = 256 rows).
  const long long tiles1 = (long long)((p.n + 127) / 128) * ((p.m + 255) / 256) * p.splitk;
  const long long tiles2 = (long long)((p.n + 255) / 256) * ((p.m + 255) / 256) * p.splitk;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // (256-row CTAs with the raw-block ring fit in shared memory for Q4_K blocks only)
  const bool wide_fits = !(p.qtype == QT_Q5_K || p.qtype == QT_Q6_K || legacy);
  const long long cost1 = ((tiles1 + sms - 1) / sms) * 840, cost2 = ((tiles2 + sms - 1) / sms) * 1100;
  const bool wide = wide_fits && (p._pad == 2 || (p._pad != 1 && cost2 < cost1));
  return wide ? launch_gemm<256, 2>(p, st) : launch_gemm<256, 1>(p, st);
}

// Diagnostics: switch the phase trace on/off; `rlz_gemm_trace_read` copies the records (GM_TRACE_PTS timestamps in ns per CTA:
// entry, set-up done, dependency wait done, first weight block landed, producer loop done, MMAs done, epilogue done).
int rlz_gemm_trace_enable(int on) {
  const int v = on ? 1 : 0;
  return (int)cudaMemcpyToSymbol(rlz::g_gemm_trace_on, &v, sizeof(int));
}
int rlz_gemm_trace_read(unsigned long long* out, int ctas) {
  if (ctas < 1 || ctas > rlz::GM_TRACE_CTAS) return -1;
  return (int)cudaMemcpyFromSymbol(out, rlz::g_gemm_trace, sizeof(unsigned long long) * ctas * rlz::GM_TRACE_PTS);
}

int rlz_sizeof_gemm_params() { return (int)sizeof(rlz::GemmParams); }

}  // extern "C"
