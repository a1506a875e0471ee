// Decode GEMV for K-quant weights (Q4_K / Q5_K / Q6_K) with the weights moved by the copy engine:
// every warp streams "its" rows of the CTA's slab into a private shared-memory ring with
// `cp.async.bulk` (completion on the warp's own mbarriers) and consumes them from there.
//
//   * The first copies are requested BEFORE the programmatic dependency wait: weights do not depend
//     on the previous kernel, so they are in flight while it drains and while this kernel
//     normalises and quantises its input.  Bytes in flight cost no registers.
//   * A lane consumes whole half-blocks (128 weights) from shared memory, so the block header and
//     the 6-bit scale decode are paid once per 128 weights, and the L lanes that share a row all
//     stay in that row: the per-row reduction is log2(L) shuffles, no selects, no shared-memory fold.
//     A warp takes passes of 32 / L rows (one bulk copy each); L is chosen per segment on the host.
//   * Warps are independent pipelines (no CTA-wide barrier between the input staging and the
//     epilogue); 256 threads per CTA, two CTAs per SM.
//   * Input staging issues the loads of x, the norm weight and the norm bias together (one memory
//     round trip), reduces the statistics from registers (two passes over registers for LayerNorm:
//     mean first, then centred squares) and writes int8 codes in a bank-swizzled natural order.
//
// Prologue features and the epilogue (bias / activation / gated combine / second accumulated
// matrix / residual / int8 hand-off / tensor-parallel all-reduce) are those of gemv.cu, which
// remains the path for 32-wide block types, dense rows and launches that do not fit the ring.
//
// Every mbarrier wait is bounded: on expiry the CTA records 1002 in the device error word, skips
// the math of that pass, drains (bounded) the copies it still has in flight and finishes.
//
// Replaces the same reference kernels as gemv.cu (src/cuda/executor/q4k_mwv_gemv.rs:7-945,
// src/cuda/executor/layers/gemv_dispatch.rs:53-309).
#include "common.cuh"
#include <stdlib.h>
#include "../gemv_units.h"
#include "../gemv_blocks.h"
#include "gemv_params.h"
#include "gemv_common.cuh"
#include "gemv_body.cuh"

namespace rlz {

__device__ int g_slab_error = 0;
                   // 1002: a weight pass never arrived

constexpr int SL_THREADS = 256, SL_WARPS = SL_THREADS / 32;
constexpr int SL_MAX_SLOTS = 3;
constexpr uint32_t SL_WAIT_LIMIT = 1u << 22;        // try_wait iterations before giving up

__device__ __forceinline__ uint32_t sl_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool sl_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(sl_smem(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool sl_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < SL_WAIT_LIMIT; ++spin)
    if (sl_try_wait(bar, parity)) return true;
  return false;
}

// position of 16-byte chunk ci of an activation row: the chunk keeps its group of eight (= one half-block of 128
// values) and its position inside the group is XOR-ed with the half-block index, so that lanes working on different half-blocks of a row
// (same relative chunk) read different bank groups
RLZ_HD int sw_chunk_off(int ci) { return ((ci & ~7) | ((ci ^ (ci >> 3)) & 7)) << 4; }

// Shared-memory activations of one input for B rows:
//   q    : int8[B][k]      codes, chunk ci at sw_chunk_off(ci)
//   rec4 : float4[B][k/64] {d[2G], d[2G+1], d[2G] * sum32[2G], d[2G+1] * sum32[2G+1]} of 64-group G (Q4_K / Q5_K)
//   rec6 : float2[B][k/16] {d of the chunk's 32-block, d * sum16 of the chunk}                (Q6_K)
struct ActSw { const int8_t* q; const U4* rec4; const F2* rec6; int k; };

__device__ __forceinline__ size_t sl_act_bytes(int B, int k) { return (size_t)B * k + (size_t)B * (k >> 6) * 16 + (size_t)B * (k >> 4) * 8; }

// ---- half-block dot products (128 weights of block hb >> 1, half hb & 1) against B activation rows ----
template <int B>
__device__ __forceinline__ void hb_q4k(const uint8_t* blk, int hb, const ActSw& a, float* acc) {
  const int h = hb & 1;
  const U4 hdr = ld_s16(blk);
  float d, dmin;
  h2f_pair(hdr.x, &d, &dmin);
  uint32_t scw, mw;                                   // scales / mins of sub-blocks 4h .. 4h+3 as packed bytes
  if (h == 0) { scw = hdr.y & 0x3F3F3F3Fu; mw = hdr.z & 0x3F3F3F3Fu; }
  else {
    scw = (hdr.w & 0x0F0F0F0Fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    mw = ((hdr.w >> 4) & 0x0F0F0F0Fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
  }
  const int8_t* xq0 = a.q + (hb << 7);
  const int sw = (hb & 7) << 4;                        // XOR swizzle of the chunk position inside the half-block
#pragma unroll
  for (int gg = 0; gg < 2; ++gg) {
    const int g = 2 * h + gg;
    const U4 q0 = ld_s16(blk + 16 + 32 * g), q1 = ld_s16(blk + 32 + 32 * g);
    const U4 lo0 = RLZ_LO4(q0), lo1 = RLZ_LO4(q1);
    // high nibbles stay in place (value * 16); the factor 1/16 goes into the scale
    const U4 hi0{q0.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q0.z & 0xF0F0F0F0u, q0.w & 0xF0F0F0F0u};
    const U4 hi1{q1.x & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u, q1.z & 0xF0F0F0F0u, q1.w & 0xF0F0F0F0u};
    const float fs0 = d * i2f((int)((scw >> (16 * gg)) & 0xFFu)), fs1 = d * 0.0625f * i2f((int)((scw >> (16 * gg + 8)) & 0xFFu));
    const float fm0 = dmin * i2f((int)((mw >> (16 * gg)) & 0xFFu)), fm1 = dmin * i2f((int)((mw >> (16 * gg + 8)) & 0xFFu));
    const int o0 = ((4 * gg) << 4) ^ sw, o1 = ((4 * gg + 1) << 4) ^ sw, o2 = ((4 * gg + 2) << 4) ^ sw, o3 = ((4 * gg + 3) << 4) ^ sw;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int8_t* xq = xq0 + (size_t)b * a.k;
      const U4 r = a.rec4[(size_t)b * (a.k >> 6) + 2 * hb + gg];
      const int dlo = dot16(lo0, ld_a16(xq + o0)) + dot16(lo1, ld_a16(xq + o1));
      const int dhi = dot16us(hi0, ld_a16(xq + o2)) + dot16us(hi1, ld_a16(xq + o3));
      acc[b] += as_f(r.x) * fs0 * i2f(dlo) - fm0 * as_f(r.z) + as_f(r.y) * fs1 * i2f(dhi) - fm1 * as_f(r.w);
    }
  }
}

template <int B>
__device__ __forceinline__ void hb_q5k(const uint8_t* blk, int hb, const ActSw& a, float* acc) {
  const int h = hb & 1;
  const U4 hdr = ld_s16(blk);
  const U4 h0 = ld_s16(blk + 16), h1 = ld_s16(blk + 32);
  float d, dmin;
  h2f_pair(hdr.x, &d, &dmin);
  uint32_t scw, mw;
  if (h == 0) { scw = hdr.y & 0x3F3F3F3Fu; mw = hdr.z & 0x3F3F3F3Fu; }
  else {
    scw = (hdr.w & 0x0F0F0F0Fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    mw = ((hdr.w >> 4) & 0x0F0F0F0Fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
  }
  const int8_t* xq0 = a.q + (hb << 7);
  const int sw = (hb & 7) << 4;                        // XOR swizzle of the chunk position inside the half-block
#pragma unroll
  for (int gg = 0; gg < 2; ++gg) {
    const int g = 2 * h + gg;
    const U4 q0 = ld_s16(blk + 48 + 32 * g), q1 = ld_s16(blk + 64 + 32 * g);
    const int s0 = 2 * g, s1 = 2 * g + 1;
#define RLZ_Q5L(qw, hw) (((qw) & 0x0F0F0F0Fu) | ((((hw) >> s0) & 0x01010101u) << 4))
#define RLZ_Q5H(qw, hw) ((((qw) >> 4) & 0x0F0F0F0Fu) | ((((hw) >> s1) & 0x01010101u) << 4))
    const U4 lo0{RLZ_Q5L(q0.x, h0.x), RLZ_Q5L(q0.y, h0.y), RLZ_Q5L(q0.z, h0.z), RLZ_Q5L(q0.w, h0.w)};
    const U4 lo1{RLZ_Q5L(q1.x, h1.x), RLZ_Q5L(q1.y, h1.y), RLZ_Q5L(q1.z, h1.z), RLZ_Q5L(q1.w, h1.w)};
    const U4 hi0{RLZ_Q5H(q0.x, h0.x), RLZ_Q5H(q0.y, h0.y), RLZ_Q5H(q0.z, h0.z), RLZ_Q5H(q0.w, h0.w)};
    const U4 hi1{RLZ_Q5H(q1.x, h1.x), RLZ_Q5H(q1.y, h1.y), RLZ_Q5H(q1.z, h1.z), RLZ_Q5H(q1.w, h1.w)};
#undef RLZ_Q5L
#undef RLZ_Q5H
    const float fs0 = d * i2f((int)((scw >> (16 * gg)) & 0xFFu)), fs1 = d * i2f((int)((scw >> (16 * gg + 8)) & 0xFFu));
    const float fm0 = dmin * i2f((int)((mw >> (16 * gg)) & 0xFFu)), fm1 = dmin * i2f((int)((mw >> (16 * gg + 8)) & 0xFFu));
    const int o0 = ((4 * gg) << 4) ^ sw, o1 = ((4 * gg + 1) << 4) ^ sw, o2 = ((4 * gg + 2) << 4) ^ sw, o3 = ((4 * gg + 3) << 4) ^ sw;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int8_t* xq = xq0 + (size_t)b * a.k;
      const U4 r = a.rec4[(size_t)b * (a.k >> 6) + 2 * hb + gg];
      const int dlo = dot16(lo0, ld_a16(xq + o0)) + dot16(lo1, ld_a16(xq + o1));
      const int dhi = dot16(hi0, ld_a16(xq + o2)) + dot16(hi1, ld_a16(xq + o3));
      acc[b] += as_f(r.x) * fs0 * i2f(dlo) - fm0 * as_f(r.z) + as_f(r.y) * fs1 * i2f(dhi) - fm1 * as_f(r.w);
    }
  }
}

// Q6_K, 224-byte device blocks: half n = weights [128n, 128n + 128)
template <int B>
__device__ __forceinline__ void hb_q6k(const uint8_t* blk, int hb, const ActSw& a, float* acc) {
  const int n = hb & 1;
  const U4 scv = ld_s16(blk + 192);
  const U4 tail = ld_s16(blk + 208);
  float d, unused;
  h2f_pair(tail.x, &d, &unused);
  const uint32_t scw0 = n ? scv.z : scv.x, scw1 = n ? scv.w : scv.y;          // the 8 scales of this half
  const int8_t* xq0 = a.q + (hb << 7);
  const int sw = (hb & 7) << 4;
#pragma unroll
  for (int lh = 0; lh < 2; ++lh) {
    const U4 qa = ld_s16(blk + n * 64 + 16 * lh), qb = ld_s16(blk + n * 64 + 32 + 16 * lh), qh = ld_s16(blk + 128 + n * 32 + 16 * lh);
    U4 w[4];
    w[0] = U4{(qa.x & 0x0F0F0F0Fu) | ((qh.x & 0x03030303u) << 4), (qa.y & 0x0F0F0F0Fu) | ((qh.y & 0x03030303u) << 4),
              (qa.z & 0x0F0F0F0Fu) | ((qh.z & 0x03030303u) << 4), (qa.w & 0x0F0F0F0Fu) | ((qh.w & 0x03030303u) << 4)};
    w[1] = U4{(qb.x & 0x0F0F0F0Fu) | (((qh.x >> 2) & 0x03030303u) << 4), (qb.y & 0x0F0F0F0Fu) | (((qh.y >> 2) & 0x03030303u) << 4),
              (qb.z & 0x0F0F0F0Fu) | (((qh.z >> 2) & 0x03030303u) << 4), (qb.w & 0x0F0F0F0Fu) | (((qh.w >> 2) & 0x03030303u) << 4)};
    w[2] = U4{((qa.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> 4) & 0x03030303u) << 4), ((qa.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> 4) & 0x03030303u) << 4),
              ((qa.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> 4) & 0x03030303u) << 4), ((qa.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> 4) & 0x03030303u) << 4)};
    w[3] = U4{((qb.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> 6) & 0x03030303u) << 4), ((qb.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> 6) & 0x03030303u) << 4),
              ((qb.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> 6) & 0x03030303u) << 4), ((qb.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> 6) & 0x03030303u) << 4)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int si = lh + 2 * j;                                              // scale index inside the half = chunk inside the half
      const float fs = d * i2f((int)(int8_t)(((si < 4 ? scw0 : scw1) >> (8 * (si & 3))) & 0xFFu));
      const int off = (si << 4) ^ sw;
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int dj = dot16(w[j], ld_a16(xq0 + (size_t)b * a.k + off));
        const F2 r = a.rec6[(size_t)b * (a.k >> 4) + 8 * hb + si];
        acc[b] += fs * (r.x * i2f(dj) - 32.f * r.y);
      }
    }
  }
}

// ---- input staging ----------------------------------------------------------------------------------------
struct SlabIn {                      // one input of the CTA's matrix, read from the parameter block before the dependency wait
  const float* x; const float* nw; const float* nb; const uint8_t* pre;
  int64_t ld; int32_t k, norm; float eps; int32_t act_off;
};

// One input row -> int8 codes + records in shared memory.  NV float4 per thread cover k <= NV * 4 * SL_THREADS.
// Needs k % 128 == 0 (a group of eight lanes = one 32-block is all inside or all outside the row).  The loads of x, the
// norm weight and the norm bias are issued together; everything after them is straight-line code over registers so that
// the shuffle chains of the NV iterations overlap.  `red` holds 2 * SL_WARPS floats.
template <int NV, class AfterLoads>
__device__ __forceinline__ void sl_stage_row(const SlabIn& X, const float* x, int8_t* q, float* rec4, float* rec6, float* red, AfterLoads&& after_loads) {
  const int k = X.k, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr bool PRELOAD = NV <= 4;                  // norm weight / bias held in registers next to x
  float4 v[NV], nw[PRELOAD ? NV : 1], nb[PRELOAD ? NV : 1];
  const bool normed = X.norm != NORM_NONE;
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int i = (it * SL_THREADS + tid) * 4;
    v[it] = i < k ? *(const float4*)(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (PRELOAD) {
      nw[it] = (normed && X.nw && i < k) ? __ldg((const float4*)(X.nw + i)) : make_float4(1.f, 1.f, 1.f, 1.f);
      nb[it] = (normed && X.nb && i < k) ? __ldg((const float4*)(X.nb + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  after_loads();                                      // the input's loads are in the memory system: later requests queue behind them
  float mean = 0.f, rstd = 1.f;
  if (normed) {
    if (X.norm == NORM_LAYER) {
      float s = 0.f;
#pragma unroll
      for (int it = 0; it < NV; ++it) s += v[it].x + v[it].y + v[it].z + v[it].w;          // padding is zero
      s = warp_sum(s);
      if (lane == 0) red[warp] = s;
      __syncthreads();
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SL_WARPS; ++w) t += red[w];
      mean = t / (float)k;
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const bool in = (it * SL_THREADS + tid) * 4 < k;
      const float a = v[it].x - mean, c = v[it].y - mean, d = v[it].z - mean, e = v[it].w - mean;
      ss += in ? a * a + c * c + d * d + e * e : 0.f;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[SL_WARPS + warp] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < SL_WARPS; ++w) t += red[SL_WARPS + w];
    rstd = rsqrtf(t / (float)k + X.eps);
  }
  float amax[NV];
#pragma unroll
  for (int it = 0; it < NV; ++it) {                  // rows past k carry zeros through the arithmetic; only their stores are skipped
    const int i = (it * SL_THREADS + tid) * 4;
    float4 w = v[it];
    if (normed) {
      w.x = (w.x - mean) * rstd; w.y = (w.y - mean) * rstd; w.z = (w.z - mean) * rstd; w.w = (w.w - mean) * rstd;
      if (PRELOAD) {
        w.x = w.x * nw[it].x + nb[it].x; w.y = w.y * nw[it].y + nb[it].y; w.z = w.z * nw[it].z + nb[it].z; w.w = w.w * nw[it].w + nb[it].w;
      } else if (i < k) {
        if (X.nw) { const float4 g = __ldg((const float4*)(X.nw + i)); w.x *= g.x; w.y *= g.y; w.z *= g.z; w.w *= g.w; }
        if (X.nb) { const float4 g = __ldg((const float4*)(X.nb + i)); w.x += g.x; w.y += g.y; w.z += g.z; w.w += g.w; }
      }
    }
    v[it] = w;
    amax[it] = fmaxf(fmaxf(fabsf(w.x), fabsf(w.y)), fmaxf(fabsf(w.z), fabsf(w.w)));
  }
#pragma unroll
  for (int o = 1; o <= 4; o <<= 1) {
#pragma unroll
    for (int it = 0; it < NV; ++it) amax[it] = fmaxf(amax[it], __shfl_xor_sync(0xffffffffu, amax[it], o));
  }
  uint32_t packed[NV];
  int s16[NV], s32[NV];
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const float inv = amax[it] > 0.f ? __fdividef(127.f, amax[it]) : 0.f;
    const int q0 = __float2int_rn(v[it].x * inv), q1 = __float2int_rn(v[it].y * inv), q2 = __float2int_rn(v[it].z * inv), q3 = __float2int_rn(v[it].w * inv);
    packed[it] = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    s16[it] = q0 + q1 + q2 + q3;
  }
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
#pragma unroll
    for (int it = 0; it < NV; ++it) s16[it] += __shfl_xor_sync(0xffffffffu, s16[it], o);
  }
#pragma unroll
  for (int it = 0; it < NV; ++it) s32[it] = s16[it] + __shfl_xor_sync(0xffffffffu, s16[it], 4);
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int i = (it * SL_THREADS + tid) * 4;
    if (i < k) {
      const float d = amax[it] * (1.f / 127.f);
      *(uint32_t*)(q + sw_chunk_off(i >> 4) + (i & 15)) = packed[it];
      if ((tid & 3) == 0) { float* r6 = rec6 + (size_t)(i >> 4) * 2; r6[0] = d; r6[1] = d * (float)s16[it]; }
      if ((tid & 7) == 0) { float* r4 = rec4 + (size_t)(i >> 6) * 4 + ((i >> 5) & 1); r4[0] = d; r4[2] = d * (float)s32[it]; }
    }
  }
}

// The producing launch left this activation quantised (GemvMat::q_out layout: codes | per-64 records | per-32 scales |
// per-16 sums): re-order the codes into this kernel's chunk order and turn the integer sums into the float records.
__device__ __forceinline__ void sl_stage_pre(const uint8_t* g, int k, int8_t* q, float* rec4, float* rec6) {
  const uint32_t* xm = (const uint32_t*)(g + k);
  const float* xd = (const float*)(g + k + (k >> 2));
  const int32_t* xs = (const int32_t*)(g + k + (k >> 2) + (k >> 3));
  for (int ci = threadIdx.x; ci < (k >> 4); ci += SL_THREADS) {
    *(uint4*)(q + sw_chunk_off(ci)) = *(const uint4*)(g + act_chunk_off(ci));
    const float d = xd[ci >> 1];
    rec6[2 * ci] = d; rec6[2 * ci + 1] = d * (float)xs[ci];
  }
  for (int G = threadIdx.x; G < (k >> 6); G += SL_THREADS) {
    const uint4 r = *(const uint4*)(xm + 4 * G);
    const float d0 = __uint_as_float(r.x), d1 = __uint_as_float(r.y);
    *(float4*)(rec4 + 4 * G) = make_float4(d0, d1, d0 * (float)(int)r.z, d1 * (float)(int)r.w);
  }
}

struct SlabLaunch {                  // host-computed geometry of a launch
  int32_t early;                     // weight copies requested before the dependency wait: 1 = this warp's first slots, 0 = none
  int32_t nomath;                    // diagnostics: wait for the weights but skip the dot products (results are wrong)
  int32_t ring_bytes;                // per warp
  int32_t slot_bytes;                // ring_bytes / nslots, a multiple of 128
  int32_t nslots;
  int32_t act_off[GEMV_MAX_X];       // byte offset of each input's activation area behind the rings (-1: input unused)
  int32_t misc_off;                  // red + rowacc
};

template <int B>
__global__ void __launch_bounds__(SL_THREADS, 2) gemv_slab_kernel(const __grid_constant__ GemvParams p, const __grid_constant__ SlabLaunch g) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[SL_WARPS][SL_MAX_SLOTS];
  __shared__ int failed_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bx = (int)blockIdx.x;
  int m = 0;
  while (m + 1 < p.nmat && bx >= p.mat[m + 1].cta_begin) ++m;
  const GemvMat& M = p.mat[m];
  const int r0 = (bx - M.cta_begin) * M.rows_per_cta;
  const int r1 = min(M.n, r0 + M.rows_per_cta);
  const int nrows = r1 - r0;

  // pass geometry of the (up to two) segments: L lanes per row, 32 / L rows per pass
  int segL[2], rpp[2], npass[2], rowb[2], bbs[2], nhb[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const bool on = s < M.nseg;
    segL[s] = on ? M.seg[s]._pad : 32;
    rpp[s] = 32 / segL[s];
    npass[s] = on ? (nrows + rpp[s] - 1) / rpp[s] : 0;
    bbs[s] = on ? dev_block_bytes(M.seg[s].qtype) : 0;
    nhb[s] = on ? M.seg[s].k >> 7 : 0;
    rowb[s] = on ? (M.seg[s].k >> 8) * bbs[s] : 0;
  }
  const int total = npass[0] + npass[1];
  const bool tr = tid == 0 && bx < GEMV_TRACE_CTAS && (g_gemv_trace_on == 1 || (g_gemv_trace_on == 2 && p._pad));   // 2: tagged launches only
  gemv_trace(tr, bx, 0);
  uint8_t* ring = smem + (size_t)warp * g.ring_bytes;
  uint64_t* bar = bars[warp];

  int issued = 0;
  auto issue_next = [&]() {                         // lane 0 only: request this warp's next pass, if any
    const int P = warp + issued * SL_WARPS;
    if (P >= total) return;
    const int s = P < npass[0] ? 0 : 1;
    const int pr0 = (P - (s ? npass[0] : 0)) * (s ? rpp[1] : rpp[0]);
    const int rows = min((s ? rpp[1] : rpp[0]), nrows - pr0);
    const uint32_t bytes = (uint32_t)rows * (uint32_t)(s ? rowb[1] : rowb[0]);
    const int slot = issued % g.nslots;
    const uint8_t* src = M.seg[s].W + (int64_t)(r0 + pr0) * M.seg[s].stride;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sl_smem(&bar[slot])), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(sl_smem(ring + (size_t)slot * g.slot_bytes)), "l"(src), "r"(bytes), "r"(sl_smem(&bar[slot])) : "memory");
    ++issued;
  };

  // the inputs of this CTA's matrix, read from the parameter block while the previous kernel still runs
  const int nin = (M.nseg == 2 && M.seg[1].x_id != M.seg[0].x_id) ? 2 : 1;
  SlabIn in0, in1;
  {
    const GemvX& X = p.xs[M.seg[0].x_id];
    in0 = SlabIn{X.x, X.nw, X.nb, X.pre, X.ld, X.k, X.norm, X.eps, g.act_off[M.seg[0].x_id]};
    const GemvX& Y = p.xs[M.seg[nin - 1].x_id];
    in1 = SlabIn{Y.x, Y.nw, Y.nb, Y.pre, Y.ld, Y.k, Y.norm, Y.eps, g.act_off[M.seg[nin - 1].x_id]};
  }

  if (tid == 0) failed_s = 0;
  if (lane == 0) {
    for (int i = 0; i < g.nslots; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sl_smem(&bar[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (g.early) for (int i = 0; i < g.nslots; ++i) issue_next();        // weights do not depend on earlier kernels
  }
  pdl_launch_dependents();
  pdl_wait();
  gemv_trace(tr, bx, 1);

  // ---- stage every input this CTA's matrix multiplies -------------------------------------------------------
  float* red = (float*)(smem + g.misc_off);
  float* rowacc = red + 2 * SL_WARPS;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (s >= nin) break;
    const SlabIn& X = s == 0 ? in0 : in1;
    const int k = X.k;
    uint8_t* base = smem + X.act_off;
    int8_t* q = (int8_t*)base;
    float* rec4 = (float*)(base + (size_t)B * k);
    float* rec6 = rec4 + (size_t)B * (k >> 6) * 4;
    if (B == 1 && X.pre) sl_stage_pre(X.pre, k, q, rec4, rec6);
    else {
#pragma unroll 1
      for (int b = 0; b < B; ++b) {
        const float* x = X.x + (int64_t)b * X.ld;
        int8_t* qb = q + (size_t)b * k;
        float* r4 = rec4 + (size_t)b * (k >> 6) * 4;
        float* r6 = rec6 + (size_t)b * (k >> 4) * 2;
        if (b > 0 || s > 0) __syncthreads();            // the statistics scratch of the previous row has been read
        auto late = [&]() { if (!g.early && lane == 0 && issued == 0) for (int i = 0; i < g.nslots; ++i) issue_next(); };
        const int nv = (k + 4 * SL_THREADS - 1) / (4 * SL_THREADS);
        switch (nv) {
          case 1: sl_stage_row<1>(X, x, qb, r4, r6, red, late); break;
          case 2: sl_stage_row<2>(X, x, qb, r4, r6, red, late); break;
          case 3: sl_stage_row<3>(X, x, qb, r4, r6, red, late); break;
          case 4: sl_stage_row<4>(X, x, qb, r4, r6, red, late); break;
          case 5: case 6: case 7: case 8: sl_stage_row<8>(X, x, qb, r4, r6, red, late); break;
          default: sl_stage_row<16>(X, x, qb, r4, r6, red, late); break;
        }
      }
    }
  }
  if (!g.early && lane == 0 && issued == 0) for (int i = 0; i < g.nslots; ++i) issue_next();      // (pre-quantised inputs only)
  __syncthreads();
  gemv_trace(tr, bx, 2);

  // ---- rows: every warp walks its own passes ------------------------------------------------------------------
  bool ok = true;
  for (int c = 0;; ++c) {
    const int P = warp + c * SL_WARPS;
    if (P >= total) break;
    const int s = P < npass[0] ? 0 : 1;
    const int slot = c % g.nslots;
    if (ok && !sl_wait(&bar[slot], (uint32_t)(c / g.nslots) & 1u)) { ok = false; failed_s = 1; atomicExch(&g_slab_error, 1002); }
    const GemvSeg& S = M.seg[s];
    const int L = (s ? segL[1] : segL[0]), rr = lane / L, sub = lane - rr * L;
    const int pr0 = (P - (s ? npass[0] : 0)) * (s ? rpp[1] : rpp[0]);
    const int row = pr0 + rr;
    const uint8_t* wrow = ring + (size_t)slot * g.slot_bytes + (size_t)rr * (s ? rowb[1] : rowb[0]);
    const uint8_t* abase = smem + g.act_off[S.x_id];
    const ActSw a{(const int8_t*)abase, (const U4*)(abase + (size_t)B * S.k), (const F2*)(abase + (size_t)B * S.k + (size_t)B * (S.k >> 6) * 16), S.k};
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.f;
    if (ok && row < nrows && !g.nomath) {
      const int n = (s ? nhb[1] : nhb[0]), bb = (s ? bbs[1] : bbs[0]);
      switch (S.qtype) {
        case QT_Q4_K: for (int hb = sub; hb < n; hb += L) hb_q4k<B>(wrow + (size_t)(hb >> 1) * bb, hb, a, acc); break;
        case QT_Q5_K: for (int hb = sub; hb < n; hb += L) hb_q5k<B>(wrow + (size_t)(hb >> 1) * bb, hb, a, acc); break;
        default:      for (int hb = sub; hb < n; hb += L) hb_q6k<B>(wrow + (size_t)(hb >> 1) * bb, hb, a, acc); break;
      }
    }
    for (int o = L >> 1; o > 0; o >>= 1) {
#pragma unroll
      for (int b = 0; b < B; ++b) acc[b] += __shfl_xor_sync(0xffffffffu, acc[b], o);
    }
    if (sub == 0 && row < nrows) {
#pragma unroll
      for (int b = 0; b < B; ++b) rowacc[(row * 2 + s) * B + b] = acc[b];
    }
    __syncwarp();                                     // every lane has finished reading the slot
    if (lane == 0 && ok) issue_next();
  }
  if (!ok && lane == 0) {
    // error path: give the copies this warp still has in flight a bounded chance to land before the shared memory is released
    for (int c = 0; c < issued; ++c) sl_wait(&bar[c % g.nslots], (uint32_t)(c / g.nslots) & 1u);
  }
  gemv_trace(tr, bx, 3);
  __syncthreads();
  gemv_trace(tr, bx, 6);
  gemv_epilogue<B>(p, M, rowacc, r0, r1);
  gemv_trace(tr, bx, 7);
}

// ---- host side -------------------------------------------------------------------------------------------------
static bool sl_kquant(int qt) { return qt == QT_Q4_K || qt == QT_Q5_K || qt == QT_Q6_K; }

// Validate and plan.  Returns 0, -20 when the launch does not qualify for this kernel, or the code of gemv_prepare.
static int slab_plan(GemvParams& p, SlabLaunch& g, int* grid_out, size_t* smem_out) {
  const int rc = gemv_prepare(p, grid_out);
  if (rc) return rc;
  if (p.any_generic) return -20;
  bool used[GEMV_MAX_X] = {false, false, false, false};
  for (int m = 0; m < p.nmat; ++m)
    for (int s = 0; s < p.mat[m].nseg; ++s) {
      const GemvSeg& S = p.mat[m].seg[s];
      if (!sl_kquant(S.qtype) || S.k % 256 || S.k > 16 * 4 * SL_THREADS) return -20;
      if (S.stride != (int64_t)(S.k / 256) * dev_block_bytes(S.qtype)) return -20;
      used[S.x_id] = true;
    }
  size_t act = 0;
  for (int i = 0; i < GEMV_MAX_X; ++i) {
    g.act_off[i] = -1;
    if (!used[i]) continue;
    g.act_off[i] = (int32_t)act;                     // relative; the ring size is added below
    act += ((size_t)p.batch * p.xs[i].k * 7 / 4 + 127) & ~(size_t)127;      // codes + k/4 + k/2 bytes of records
  }
  const size_t misc = (size_t)(2 * SL_WARPS) * 4 + (size_t)p.max_rows * 2 * p.batch * 4;
  const size_t budget = 113 * 1024 - 512;            // two CTAs per SM (static shared memory and the per-CTA reserve come on top)
  if (act + misc + 128 > budget) return -20;
  int ring = (int)((budget - act - misc - 128) / SL_WARPS) & ~127;
  if (ring > 32 * 1024) ring = 32 * 1024;
  // lanes per row of every segment: the fewest serial half-blocks per lane over the rounds of passes that fit a ring slot
  int max_pass = 0;
  for (int m = 0; m < p.nmat; ++m) {
    GemvMat& M = p.mat[m];
    for (int s = 0; s < M.nseg; ++s) {
      GemvSeg& S = M.seg[s];
      const int rowb = (S.k / 256) * dev_block_bytes(S.qtype), nhb = S.k / 128;
      int best = 0, best_cost = 1 << 30;
      for (int L = 2; L <= 32; L <<= 1) {
        const int rows = 32 / L;
        if (rows * rowb > ring) continue;
        const int np = (M.rows_per_cta + rows - 1) / rows;
        const int cost = ((np + SL_WARPS - 1) / SL_WARPS) * ((nhb + L - 1) / L);
        if (cost < best_cost) { best_cost = cost; best = L; }       // ties keep the smaller L (more rows per copy)
      }
      if (!best) return -20;
      S._pad = best;
      const int pass = (32 / best) * rowb;
      if (pass > max_pass) max_pass = pass;
    }
  }
  const int slot = (max_pass + 127) & ~127;
  int nslots = ring / slot;
  if (nslots < 1) return -20;
  if (nslots > SL_MAX_SLOTS) nslots = SL_MAX_SLOTS;
  g.nslots = nslots; g.slot_bytes = slot; g.ring_bytes = nslots * slot;
  static const int early_env = [] { const char* e = getenv("RLZ_SLAB_EARLY"); return e ? atoi(e) : 1; }();
  g.early = early_env;
  static const int nomath_env = [] { const char* e = getenv("RLZ_SLAB_NOMATH"); return e ? atoi(e) : 0; }();
  g.nomath = nomath_env;
  const size_t rings = (size_t)SL_WARPS * g.ring_bytes;
  for (int i = 0; i < GEMV_MAX_X; ++i) if (g.act_off[i] >= 0) g.act_off[i] += (int32_t)rings;
  g.misc_off = (int32_t)((rings + act + 15) & ~(size_t)15);
  *smem_out = (size_t)g.misc_off + misc;
  return 0;
}

template <int B>
static cudaError_t launch_slab(const GemvParams& p, const SlabLaunch& g, int grid, size_t smem, cudaStream_t stream) {
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(gemv_slab_kernel<B>, 113 * 1024); e != cudaSuccess) return e;
  return launch(gemv_slab_kernel<B>, dim3(grid), dim3(SL_THREADS), smem, stream, p, g);
}

}  // namespace rlz

extern "C" {

// 0 / error code recorded by a CTA whose bounded wait for a weight pass expired (1002)
int rlz_gemv_slab_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, rlz::g_slab_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) { int z = 0; cudaMemcpyToSymbol(rlz::g_slab_error, &z, sizeof(int)); }
  return v;
}

// Diagnostics: phase trace of this kernel, same record layout as rlz_gemv_trace_read (entry, dependency wait done, inputs staged,
// warp 0's rows done, all rows done, epilogue done).
int rlz_gemv_slab_trace_enable(int on) {
  const int v = on;                                  // 1: every launch, 2: launches whose parameter block is tagged (_pad != 0)
  return (int)cudaMemcpyToSymbol(rlz::g_gemv_trace_on, &v, sizeof(int));
}
int rlz_gemv_slab_trace_read(unsigned long long* out, int ctas, int clear) {
  if (ctas < 1 || ctas > rlz::GEMV_TRACE_CTAS) return -1;
  cudaError_t e = cudaMemcpyFromSymbol(out, rlz::g_gemv_trace, sizeof(unsigned long long) * ctas * rlz::GEMV_TRACE_PTS);
  if (e != cudaSuccess || !clear) return (int)e;
  static unsigned long long zeros[rlz::GEMV_TRACE_CTAS * rlz::GEMV_TRACE_PTS];
  return (int)cudaMemcpyToSymbol(rlz::g_gemv_trace, zeros, sizeof(zeros));
}

// 0 when rlz_gemv_slab would take this launch, -20 when it does not qualify, another negative code for invalid parameters.
int rlz_gemv_slab_check(const rlz::GemvParams* pp) {
  using namespace rlz;
  GemvParams p = *pp;
  SlabLaunch g;
  int grid = 0; size_t smem = 0;
  return slab_plan(p, g, &grid, &smem);
}

// Same parameter block and return convention as rlz_gemv; -20 when the launch does not qualify (K-quant segments with
// k % 256 == 0 and contiguous rows whose activations and at least one pass per warp fit half an SM's shared memory).
int rlz_gemv_slab(const rlz::GemvParams* pp, void* stream) {
  using namespace rlz;
  GemvParams p = *pp;
  SlabLaunch g;
  int grid = 0; size_t smem = 0;
  const int rc = slab_plan(p, g, &grid, &smem);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  switch (p.batch) {
    case 1: e = launch_slab<1>(p, g, grid, smem, st); break;
    case 2: e = launch_slab<2>(p, g, grid, smem, st); break;
    case 3: e = launch_slab<3>(p, g, grid, smem, st); break;
    default: e = launch_slab<4>(p, g, grid, smem, st); break;
  }
  return (int)e;
}

}  // extern "C"
