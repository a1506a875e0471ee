// Whole-super-block dot products for the streamed decode GEMV (kernels/gemv_stream.cu): one lane
// consumes one 256-weight K-quant block (already staged in shared memory by a bulk copy) against
// int8 activations, so the scale decode, addressing and bookkeeping are paid once per 256
// weights.  Host/device code, like gemv_units.h, so the bit manipulation is testable on a CPU.
//
// Two lanes share a block: each takes one half (128 weights).
//
// Activation layout in shared memory for B rows (row strides derived from k, k % 256 == 0,
// nsb = k / 256).  Everything is stored "chunk-major" so that lanes working on consecutive
// super-blocks read consecutive addresses:
//   q    : int8[k]     the 16-byte chunk c (0..15) of super-block sb sits at (c * nsb + sb) * 16
//   rec4 : float4[k/64] record (g * nsb + sb) = {d[2g], d[2g+1], d*sum32[2g], d*sum32[2g+1]} of sb
//                       (Q4_K / Q5_K: scales and min-term sums of the two 32-blocks of group g)
//   rec6 : float2[k/16] record (c * nsb + sb) = {d of the chunk's 32-block, d * sum16 of chunk c}
//                       (Q6_K: scale and offset-term sum of every 16-value chunk)
#pragma once
#include "gemv_units.h"

namespace rlz {

struct F2 { float x, y; };
struct ActBlk {
  const int8_t* q; const U4* rec4; const F2* rec6; int k; int nsb;
};

RLZ_HD int blk_chunk_off(int nsb, int sb, int c) { return (c * nsb + sb) << 4; }

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ U4 ld_s16(const uint8_t* p) { const uint4 t = *(const uint4*)p; U4 v{t.x, t.y, t.z, t.w}; return v; }
#else
inline U4 ld_s16(const uint8_t* p) { U4 v; memcpy(&v, p, 16); return v; }
#endif

// all eight 6-bit scales / mins of a Q4_K / Q5_K block as packed bytes
struct K4Scales { uint32_t sc_lo, sc_hi, m_lo, m_hi; };
RLZ_HD K4Scales k4_unpack(uint32_t y, uint32_t z, uint32_t w) {
  K4Scales s;
  s.sc_lo = y & 0x3F3F3F3Fu;
  s.m_lo = z & 0x3F3F3F3Fu;
  s.sc_hi = (w & 0x0F0F0F0Fu) | (((y >> 6) & 0x03030303u) << 4);
  s.m_hi = ((w >> 4) & 0x0F0F0F0Fu) | (((z >> 6) & 0x03030303u) << 4);
  return s;
}
RLZ_HD int k4_pick(uint32_t lo, uint32_t hi, int j) { return (int)(((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu); }

// ---- Q4_K: half h covers groups g = 2h, 2h+1 ------------------------------------------------------
template <int B>
RLZ_HD void halfblock_q4k(const uint8_t* blk, int sb, int h, const ActBlk& a, float* acc) {
  const U4 hdr = ld_s16(blk);
  const float d = h2f_alu(hdr.x & 0xFFFFu), dmin = h2f_alu(hdr.x >> 16);
  const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
  // scales / mins of sub-blocks 4h .. 4h+3 as packed bytes
  const uint32_t scw = h ? ks.sc_hi : ks.sc_lo, mw = h ? ks.m_hi : ks.m_lo;
  const int cs = a.nsb << 4;                           // byte stride between consecutive chunks
  const int8_t* xq0 = a.q + ((8 * h * a.nsb + sb) << 4);
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
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int8_t* xq = xq0 + (int64_t)b * a.k + 4 * gg * cs;
      const U4 r = a.rec4[(int64_t)b * (a.k >> 6) + g * a.nsb + sb];
      const int dlo = dot16(lo0, ld_a16(xq)) + dot16(lo1, ld_a16(xq + cs));
      const int dhi = dot16us(hi0, ld_a16(xq + 2 * cs)) + dot16us(hi1, ld_a16(xq + 3 * cs));
      acc[b] += as_f(r.x) * fs0 * i2f(dlo) - fm0 * as_f(r.z) + as_f(r.y) * fs1 * i2f(dhi) - fm1 * as_f(r.w);
    }
  }
}

// ---- Q5_K -------------------------------------------------------------------------------------
template <int B>
RLZ_HD void halfblock_q5k(const uint8_t* blk, int sb, int h, const ActBlk& a, float* acc) {
  const U4 hdr = ld_s16(blk);
  const U4 h0 = ld_s16(blk + 16), h1 = ld_s16(blk + 32);
  const float d = h2f_alu(hdr.x & 0xFFFFu), dmin = h2f_alu(hdr.x >> 16);
  const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
  const uint32_t scw = h ? ks.sc_hi : ks.sc_lo, mw = h ? ks.m_hi : ks.m_lo;
  const int cs = a.nsb << 4;
  const int8_t* xq0 = a.q + ((8 * h * a.nsb + sb) << 4);
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
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int8_t* xq = xq0 + (int64_t)b * a.k + 4 * gg * cs;
      const U4 r = a.rec4[(int64_t)b * (a.k >> 6) + g * a.nsb + sb];
      const int dlo = dot16(lo0, ld_a16(xq)) + dot16(lo1, ld_a16(xq + cs));
      const int dhi = dot16(hi0, ld_a16(xq + 2 * cs)) + dot16(hi1, ld_a16(xq + 3 * cs));
      acc[b] += as_f(r.x) * fs0 * i2f(dlo) - fm0 * as_f(r.z) + as_f(r.y) * fs1 * i2f(dhi) - fm1 * as_f(r.w);
    }
  }
}

// ---- Q6_K (224-byte device blocks): half n = weights [128n, 128n+128) --------------------------------
template <int B>
RLZ_HD void halfblock_q6k(const uint8_t* blk, int sb, int n, const ActBlk& a, float* acc) {
  const U4 scv = ld_s16(blk + 192);
  const U4 tail = ld_s16(blk + 208);
  const float d = h2f_alu(tail.x & 0xFFFFu);
  const uint32_t scw0 = n ? scv.z : scv.x, scw1 = n ? scv.w : scv.y;          // the 8 scales of this half
  const int cs = a.nsb << 4;
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
      const int si = lh + 2 * j;                                              // scale index inside the half
      const float fs = d * i2f((int)(int8_t)(((si < 4 ? scw0 : scw1) >> (8 * (si & 3))) & 0xFFu));
      const int c = n * 8 + 2 * j + lh;                                       // 16-value chunk inside the block
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int dj = dot16(w[j], ld_a16(a.q + (int64_t)b * a.k + c * cs + (sb << 4)));
        const F2 r = a.rec6[(int64_t)b * (a.k >> 4) + c * a.nsb + sb];
        acc[b] += fs * (r.x * i2f(dj) - 32.f * r.y);
      }
    }
  }
}

template <int QT, int B>
RLZ_HD void halfblock_dot(const uint8_t* blk, int sb, int h, const ActBlk& a, float* acc) {
  if (QT == QT_Q4_K) halfblock_q4k<B>(blk, sb, h, a, acc);
  else if (QT == QT_Q5_K) halfblock_q5k<B>(blk, sb, h, a, acc);
  else halfblock_q6k<B>(blk, sb, h, a, acc);
}

RLZ_HD int dev_block_bytes(int qtype) { return qtype == QT_Q4_K ? 144 : qtype == QT_Q5_K ? 176 : qtype == QT_Q6_K ? Q6K_DEV_STRIDE : 0; }

// host form of the activation staging (the kernel computes the same values cooperatively)
inline void quantize_act_row_blk(const float* v, int k, int8_t* q, U4* rec4, F2* rec6) {
  const int nsb = k / 256;
  for (int blk = 0; blk < k / 32; ++blk) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) { float a = fabsf(v[blk * 32 + i]); if (a > amax) amax = a; }
    const float dd = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
    int sum[2] = {0, 0};
    for (int i = 0; i < 32; ++i) {
      const int qi = (int)lrintf(v[blk * 32 + i] * inv);
      const int e = blk * 32 + i;
      q[blk_chunk_off(nsb, e >> 8, (e >> 4) & 15) + (e & 15)] = (int8_t)qi;
      sum[i >> 4] += qi;
    }
    const int sb = blk >> 3, j = blk & 7, g = j >> 1;
    U4& r = rec4[g * nsb + sb];
    if (j & 1) { r.y = as_u(dd); r.w = as_u(dd * (float)(sum[0] + sum[1])); } else { r.x = as_u(dd); r.z = as_u(dd * (float)(sum[0] + sum[1])); }
    for (int hh = 0; hh < 2; ++hh) { F2& r6 = rec6[(2 * j + hh) * nsb + sb]; r6.x = dd; r6.y = dd * (float)sum[hh]; }
  }
}

}  // namespace rlz
