// Integer dot "units" of the decode GEMV: each unit is what one GPU lane consumes per step —
// 16 bytes (Q6_K: 3 x 16 bytes) of quantised weights in the device layout, multiplied with
// int8-quantised activations through dp4a, for B activation rows at once.
//
// The functions compile for both host and device so that the exact bit manipulation the
// kernel runs can be checked on a CPU against the plain block decoders.
//
// Device weight layouts (rows start 16-byte aligned, `stride` bytes apart):
//   Q4_K  : ggml blocks as stored, 144 B per 256 weights
//   Q5_K  : ggml blocks as stored, 176 B per 256 weights
//   Q6_K  : ggml block followed by 14 pad bytes, 224 B per 256 weights (keeps 16-B alignment)
//   Q8_0  : planar row: [f16 d x nb, padded to 16 B][32 x i8 per block]
//   Q4_0  : planar row: [f16 d x nb, padded to 16 B][16 B nibbles per block]
// Activations: xq int8[K], xd float[K/32] (scale per 32), xs float[K/16] (= xd * sum of the 16 ints).
#pragma once
#include "quant_blocks.h"
#include <math.h>

namespace rlz {

struct U4 { uint32_t x, y, z, w; };

constexpr int Q6K_DEV_STRIDE = 224;

RLZ_HD int dev_planar_qoff(int nb) { return (2 * nb + 15) & ~15; }

// bytes per row in the device layout
RLZ_HD int64_t dev_row_bytes(int qtype, int64_t k) {
  switch (qtype) {
    case QT_Q4_K: return k / 256 * 144;
    case QT_Q5_K: return k / 256 * 176;
    case QT_Q6_K: return k / 256 * Q6K_DEV_STRIDE;
    case QT_Q8_0: return dev_planar_qoff((int)(k / 32)) + k;
    case QT_Q4_0: return dev_planar_qoff((int)(k / 32)) + k / 2;
    case QT_F32: return (k * 4 + 15) & ~(int64_t)15;
    case QT_F16: case QT_BF16: return (k * 2 + 15) & ~(int64_t)15;
    default: return ((int64_t)(k / qtype_block_elems(qtype)) * qtype_block_bytes(qtype) + 15) & ~(int64_t)15;
  }
}

// units (lane work items) per row for the int8 fast path; 0 = not a fast-path type
RLZ_HD int dev_units_per_row(int qtype, int k) {
  switch (qtype) {
    case QT_Q4_K: case QT_Q5_K: case QT_Q6_K: return k / 64;
    case QT_Q8_0: return k / 16;
    case QT_Q4_0: return k / 32;
    default: return 0;
  }
}

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ U4 ld_w16(const uint8_t* p) {   // streaming weight load: read once
  U4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ U4 ld_c16(const uint8_t* p) {   // cached load (headers shared by lanes)
  const uint4 t = __ldg((const uint4*)p); U4 v{t.x, t.y, t.z, t.w}; return v;
}
__device__ __forceinline__ U4 ld_a16(const int8_t* p) {    // activations (shared memory)
  const uint4 t = *(const uint4*)p; U4 v{t.x, t.y, t.z, t.w}; return v;
}
__device__ __forceinline__ int dp4(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }
#else
inline U4 ld_w16(const uint8_t* p) { U4 v; memcpy(&v, p, 16); return v; }
inline U4 ld_c16(const uint8_t* p) { U4 v; memcpy(&v, p, 16); return v; }
inline U4 ld_a16(const int8_t* p) { U4 v; memcpy(&v, p, 16); return v; }
inline int dp4(uint32_t a, uint32_t b, int c) {
  for (int i = 0; i < 4; ++i) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
}
inline float h2f(uint32_t bits) { return half_bits_to_float((uint16_t)bits); }
#endif

RLZ_HD int dot16(const U4& w, const U4& a) { return dp4(w.w, a.w, dp4(w.z, a.z, dp4(w.y, a.y, dp4(w.x, a.x, 0)))); }
// unsigned bytes of a times signed bytes of b
#if defined(__CUDA_ARCH__)
__device__ __forceinline__ int dp4us(uint32_t a, uint32_t b, int c) {
  int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
#else
inline int dp4us(uint32_t a, uint32_t b, int c) {
  for (int i = 0; i < 4; ++i) c += (int)(uint8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
}
#endif
RLZ_HD int dot16us(const U4& w, const U4& a) { return dp4us(w.w, a.w, dp4us(w.z, a.z, dp4us(w.y, a.y, dp4us(w.x, a.x, 0)))); }

// byte i (0..11) of the 12 packed scale bytes held in three words
RLZ_HD uint32_t k4_byte(uint32_t y, uint32_t z, uint32_t w, int i) {
  const uint32_t word = i < 4 ? y : (i < 8 ? z : w);
  return (word >> (8 * (i & 3))) & 0xFFu;
}
RLZ_HD void k4_scale_min(uint32_t y, uint32_t z, uint32_t w, int j, float* sc, float* m) {
  uint32_t s, mm;
  if (j < 4) { s = k4_byte(y, z, w, j) & 63u; mm = k4_byte(y, z, w, j + 4) & 63u; }
  else {
    const uint32_t hi = k4_byte(y, z, w, j + 4);
    s = (hi & 0xFu) | ((k4_byte(y, z, w, j - 4) >> 6) << 4);
    mm = (hi >> 4) | ((k4_byte(y, z, w, j) >> 6) << 4);
  }
  *sc = (float)s; *m = (float)mm;
}

// Activations of B rows in shared memory.  Layout per row (strides derived from k):
//   q : int8[k], stored in 16-byte chunks whose position inside each group of four chunks is
//       rotated by (chunk >> 3) so that lanes reading 64-byte-strided chunks hit distinct banks
//   d : float[k/32]  scale of each 32-block
//   s : int32[k/16]  sum of the 16 ints of each 16-chunk
//   m : 16 bytes per 64 values {d[2i], d[2i+1], sum32[2i], sum32[2i+1]} for the K-quant units
struct ActView {
  const int8_t* q; const float* d; const int32_t* s; const U4* m; int k;
};

RLZ_HD int act_chunk_off(int chunk) { return ((chunk & ~3) | ((chunk + (chunk >> 3)) & 3)) << 4; }

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ float as_f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t as_u(float f) { return __float_as_uint(f); }
#else
inline float as_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
inline uint32_t as_u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
#endif
// int -> float for |i| < 2^22 without the conversion unit: 1.5 * 2^23 + i is exact
RLZ_HD float i2f(int i) { return as_f(0x4B400000u + (uint32_t)i) - 12582912.0f; }
// fp16 bits -> float with integer ops and one multiply (exact for zero, subnormals and normals)
// the two fp16 halves of a word -> floats: one packed conversion on the device (the host form is the exact integer version)
RLZ_HD void h2f_pair(uint32_t w, float* lo, float* hi);
RLZ_HD float h2f_alu(uint32_t h) {
  const float mag = as_f((h & 0x7FFFu) << 13) * 5.192296858534828e33f;   // * 2^112
  return as_f(as_u(mag) | ((h & 0x8000u) << 16));
}
RLZ_HD void h2f_pair(uint32_t w, float* lo, float* hi) {
#if defined(__CUDA_ARCH__)
  float2 f;
  asm("{\n.reg .b16 l, h;\nmov.b32 {l, h}, %2;\ncvt.f32.f16 %0, l;\ncvt.f32.f16 %1, h;\n}" : "=f"(f.x), "=f"(f.y) : "r"(w));
  *lo = f.x; *hi = f.y;
#else
  *lo = h2f_alu(w & 0xFFFFu); *hi = h2f_alu(w >> 16);
#endif
}

RLZ_HD void k4_scale_min_i(uint32_t y, uint32_t z, uint32_t w, int j, int* sc, int* m) {
  uint32_t s, mm;
  if (j < 4) { s = k4_byte(y, z, w, j) & 63u; mm = k4_byte(y, z, w, j + 4) & 63u; }
  else {
    const uint32_t hi = k4_byte(y, z, w, j + 4);
    s = (hi & 0xFu) | ((k4_byte(y, z, w, j - 4) >> 6) << 4);
    mm = (hi >> 4) | ((k4_byte(y, z, w, j) >> 6) << 4);
  }
  *sc = (int)s; *m = (int)mm;
}

// scales and mins of the two sub-blocks 2g, 2g + 1 of a Q4_K / Q5_K block in one go: both live in the same 16-bit half of the
// three scale words, so the 6-bit fields are unpacked two at a time (a third of the instructions of two k4_scale_min_i calls,
// with no divergence between lanes that work on different groups)
RLZ_HD void k4_scale_min_pair(uint32_t y, uint32_t z, uint32_t w, int g, int* sc0, int* m0, int* sc1, int* m1) {
  const int sh = (g & 1) << 4;
  const uint32_t a2 = y >> sh, b2 = z >> sh, c2 = w >> sh;
  const uint32_t sc_lo = a2 & 0x3F3Fu, m_lo = b2 & 0x3F3Fu;
  const uint32_t sc_hi = (c2 & 0x0F0Fu) | (((a2 >> 6) & 0x0303u) << 4), m_hi = ((c2 >> 4) & 0x0F0Fu) | (((b2 >> 6) & 0x0303u) << 4);
  const uint32_t scp = (g & 2) ? sc_hi : sc_lo, mp = (g & 2) ? m_hi : m_lo;
  *sc0 = (int)(scp & 0xFFu); *sc1 = (int)((scp >> 8) & 0xFFu);
  *m0 = (int)(mp & 0xFFu); *m1 = (int)((mp >> 8) & 0xFFu);
}

#define RLZ_LO4(v) U4{(v).x & 0x0F0F0F0Fu, (v).y & 0x0F0F0F0Fu, (v).z & 0x0F0F0F0Fu, (v).w & 0x0F0F0F0Fu}
#define RLZ_HI4(v) U4{((v).x >> 4) & 0x0F0F0F0Fu, ((v).y >> 4) & 0x0F0F0F0Fu, ((v).z >> 4) & 0x0F0F0F0Fu, ((v).w >> 4) & 0x0F0F0F0Fu}

// ---- Q4_K: unit u = one 64-weight group g of a super-block (32 bytes of nibbles): low nibbles
// are sub-block 2g, high nibbles sub-block 2g+1, so one scale decode serves 64 weights ----------
template <int B>
RLZ_HD void unit_q4k(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int sb = u >> 2, g = u & 3;
  const uint8_t* base = row + (int64_t)sb * 144;
  const U4 hdr = ld_c16(base);
  const U4 q0 = ld_w16(base + 16 + 32 * g), q1 = ld_w16(base + 32 + 32 * g);
  float d, dmin;
  h2f_pair(hdr.x, &d, &dmin);
  int sc0, m0, sc1, m1;
  k4_scale_min_pair(hdr.y, hdr.z, hdr.w, g, &sc0, &m0, &sc1, &m1);
  // high nibbles stay where they are (value * 16, as unsigned bytes): their dot product is an exact multiple of 16
  const U4 lo0 = RLZ_LO4(q0), lo1 = RLZ_LO4(q1);
  const U4 hi0{q0.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q0.z & 0xF0F0F0F0u, q0.w & 0xF0F0F0F0u};
  const U4 hi1{q1.x & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u, q1.z & 0xF0F0F0F0u, q1.w & 0xF0F0F0F0u};
  // the unit's four 16-byte activation chunks 4u .. 4u + 3 (act_chunk_off of each, with the shared parts computed once)
  const int ob = u << 6, rot = u >> 1;
  const int o0 = ob | ((rot & 3) << 4), o1 = ob | (((rot + 1) & 3) << 4), o2 = ob | (((rot + 2) & 3) << 4), o3 = ob | (((rot + 3) & 3) << 4);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const U4 mm = *(const U4*)((const uint8_t*)(a.m + (int64_t)b * (a.k >> 6) + u));
    const int dlo = dot16(lo0, ld_a16(xq + o0)) + dot16(lo1, ld_a16(xq + o1));
    const int dhi = (dot16us(hi0, ld_a16(xq + o2)) + dot16us(hi1, ld_a16(xq + o3))) >> 4;
    const float t0 = d * i2f(sc0 * dlo) - dmin * i2f(m0 * (int)mm.z);
    const float t1 = d * i2f(sc1 * dhi) - dmin * i2f(m1 * (int)mm.w);
    acc[b] += as_f(mm.x) * t0 + as_f(mm.y) * t1;
  }
}

// ---- Q5_K: as Q4_K plus the fifth bit from qh (bit 2g / 2g+1 of qh[l]) ------------------------
template <int B>
RLZ_HD void unit_q5k(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int sb = u >> 2, g = u & 3;
  const uint8_t* base = row + (int64_t)sb * 176;
  const U4 hdr = ld_c16(base);
  const U4 h0 = ld_c16(base + 16), h1 = ld_c16(base + 32);
  const U4 q0 = ld_w16(base + 48 + 32 * g), q1 = ld_w16(base + 64 + 32 * g);
  float d, dmin;
  h2f_pair(hdr.x, &d, &dmin);
  int sc0, m0, sc1, m1;
  k4_scale_min_pair(hdr.y, hdr.z, hdr.w, g, &sc0, &m0, &sc1, &m1);
  const int s0 = 2 * g, s1 = 2 * g + 1;
#define RLZ_Q5(qw, hw, sh, hi) ((((hi) ? ((qw) >> 4) : (qw)) & 0x0F0F0F0Fu) | ((((hw) >> (sh)) & 0x01010101u) << 4))
  const U4 lo0{RLZ_Q5(q0.x, h0.x, s0, 0), RLZ_Q5(q0.y, h0.y, s0, 0), RLZ_Q5(q0.z, h0.z, s0, 0), RLZ_Q5(q0.w, h0.w, s0, 0)};
  const U4 hi0{RLZ_Q5(q0.x, h0.x, s1, 1), RLZ_Q5(q0.y, h0.y, s1, 1), RLZ_Q5(q0.z, h0.z, s1, 1), RLZ_Q5(q0.w, h0.w, s1, 1)};
  const U4 lo1{RLZ_Q5(q1.x, h1.x, s0, 0), RLZ_Q5(q1.y, h1.y, s0, 0), RLZ_Q5(q1.z, h1.z, s0, 0), RLZ_Q5(q1.w, h1.w, s0, 0)};
  const U4 hi1{RLZ_Q5(q1.x, h1.x, s1, 1), RLZ_Q5(q1.y, h1.y, s1, 1), RLZ_Q5(q1.z, h1.z, s1, 1), RLZ_Q5(q1.w, h1.w, s1, 1)};
#undef RLZ_Q5
  // the unit's four 16-byte activation chunks 4u .. 4u + 3 (act_chunk_off of each, with the shared parts computed once)
  const int ob = u << 6, rot = u >> 1;
  const int o0 = ob | ((rot & 3) << 4), o1 = ob | (((rot + 1) & 3) << 4), o2 = ob | (((rot + 2) & 3) << 4), o3 = ob | (((rot + 3) & 3) << 4);
  const float fs0 = d * i2f(sc0), fs1 = d * i2f(sc1);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const U4 mm = *(const U4*)((const uint8_t*)(a.m + (int64_t)b * (a.k >> 6) + u));
    const int dlo = dot16(lo0, ld_a16(xq + o0)) + dot16(lo1, ld_a16(xq + o1));
    const int dhi = dot16(hi0, ld_a16(xq + o2)) + dot16(hi1, ld_a16(xq + o3));
    const float t0 = fs0 * i2f(dlo) - dmin * i2f(m0 * (int)mm.z);
    const float t1 = fs1 * i2f(dhi) - dmin * i2f(m1 * (int)mm.w);
    acc[b] += as_f(mm.x) * t0 + as_f(mm.y) * t1;
  }
}

// ---- Q6_K (224-byte device blocks): unit u covers 4 x 16 weights of one 128-half ------------
template <int B>
RLZ_HD void unit_q6k(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int sb = u >> 2, t = u & 3, n = t >> 1, lh = t & 1;
  const uint8_t* base = row + (int64_t)sb * Q6K_DEV_STRIDE;
  const U4 qa = ld_w16(base + n * 64 + 16 * lh);
  const U4 qb = ld_w16(base + n * 64 + 32 + 16 * lh);
  const U4 qh = ld_w16(base + 128 + n * 32 + 16 * lh);
  const U4 scv = ld_c16(base + 192);
  const U4 tail = ld_c16(base + 208);
  float d, d_unused;
  h2f_pair(tail.x, &d, &d_unused);
  const uint32_t scw0 = n ? scv.z : scv.x, scw1 = n ? scv.w : scv.y;   // 8 scales of this half
  // scales lh, lh + 2, lh + 4, lh + 6 of the half: bytes lh and lh + 2 of each word (one shift per word, then fixed positions)
  const uint32_t t0 = scw0 >> (8 * lh), t1 = scw1 >> (8 * lh);
  float sc[4];
  sc[0] = d * i2f((int)(int8_t)(t0 & 0xFFu));
  sc[1] = d * i2f((int)(int8_t)((t0 >> 16) & 0xFFu));
  sc[2] = d * i2f((int)(int8_t)(t1 & 0xFFu));
  sc[3] = d * i2f((int)(int8_t)((t1 >> 16) & 0xFFu));
  U4 w[4];
  w[0] = U4{(qa.x & 0x0F0F0F0Fu) | ((qh.x & 0x03030303u) << 4), (qa.y & 0x0F0F0F0Fu) | ((qh.y & 0x03030303u) << 4),
            (qa.z & 0x0F0F0F0Fu) | ((qh.z & 0x03030303u) << 4), (qa.w & 0x0F0F0F0Fu) | ((qh.w & 0x03030303u) << 4)};
  w[1] = U4{(qb.x & 0x0F0F0F0Fu) | (((qh.x >> 2) & 0x03030303u) << 4), (qb.y & 0x0F0F0F0Fu) | (((qh.y >> 2) & 0x03030303u) << 4),
            (qb.z & 0x0F0F0F0Fu) | (((qh.z >> 2) & 0x03030303u) << 4), (qb.w & 0x0F0F0F0Fu) | (((qh.w >> 2) & 0x03030303u) << 4)};
  w[2] = U4{((qa.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> 4) & 0x03030303u) << 4), ((qa.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> 4) & 0x03030303u) << 4),
            ((qa.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> 4) & 0x03030303u) << 4), ((qa.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> 4) & 0x03030303u) << 4)};
  w[3] = U4{((qb.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> 6) & 0x03030303u) << 4), ((qb.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> 6) & 0x03030303u) << 4),
            ((qb.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> 6) & 0x03030303u) << 4), ((qb.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> 6) & 0x03030303u) << 4)};
  const int kb = sb * 256 + n * 128 + 16 * lh;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const float* xd = a.d + (int64_t)b * (a.k >> 5);
    const int32_t* xs = a.s + (int64_t)b * (a.k >> 4);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = kb + 32 * j;
      const int dj = dot16(w[j], ld_a16(xq + act_chunk_off(kk >> 4))) - 32 * xs[kk >> 4];
      sum += sc[j] * xd[kk >> 5] * i2f(dj);
    }
    acc[b] += sum;
  }
}

// ---- Q8_0 planar: unit u = 16 weights of block u/2 ------------------------------------------
template <int B>
RLZ_HD void unit_q8_0(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int nb = a.k >> 5, blk = u >> 1;
  const float d = h2f_alu((uint32_t)load_u16(row + 2 * blk));
  const U4 w = ld_w16(row + dev_planar_qoff(nb) + 16 * u);
  const int off = act_chunk_off(u);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int dj = dot16(w, ld_a16(a.q + (int64_t)b * a.k + off));
    acc[b] += d * a.d[(int64_t)b * nb + blk] * i2f(dj);
  }
}

// ---- Q4_0 planar: unit u = block u (low nibbles -> elems 0..15, high -> 16..31) -------------
template <int B>
RLZ_HD void unit_q4_0(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int nb = a.k >> 5;
  const float d = h2f_alu((uint32_t)load_u16(row + 2 * u));
  const U4 qs = ld_w16(row + dev_planar_qoff(nb) + 16 * u);
  const U4 lo = RLZ_LO4(qs), hi = RLZ_HI4(qs);
  const int o0 = act_chunk_off(2 * u), o1 = act_chunk_off(2 * u + 1);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const int32_t* xs = a.s + (int64_t)b * (a.k >> 4);
    const int dj = dot16(lo, ld_a16(xq + o0)) + dot16(hi, ld_a16(xq + o1)) - 8 * (xs[2 * u] + xs[2 * u + 1]);
    acc[b] += d * a.d[(int64_t)b * nb + u] * i2f(dj);
  }
}

template <int QT, int B>
RLZ_HD void unit_dot(const uint8_t* row, int u, const ActView& a, float* acc) {
  if (QT == QT_Q4_K) unit_q4k<B>(row, u, a, acc);
  else if (QT == QT_Q5_K) unit_q5k<B>(row, u, a, acc);
  else if (QT == QT_Q6_K) unit_q6k<B>(row, u, a, acc);
  else if (QT == QT_Q8_0) unit_q8_0<B>(row, u, a, acc);
  else if (QT == QT_Q4_0) unit_q4_0<B>(row, u, a, acc);
}

// Activation quantisation of one row (host form; the kernel does the same arithmetic
// cooperatively): per 32-block q = rint(v * 127/amax), d = amax/127; integer sums per 16.
// Output arrays follow the ActView layout (k must be a multiple of 64 for the `m` records,
// which are only filled for complete 64-groups).
inline void quantize_act_row(const float* v, int k, int8_t* q, float* d, int32_t* s16, U4* m) {
  for (int blk = 0; blk < k / 32; ++blk) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) { float a = fabsf(v[blk * 32 + i]); if (a > amax) amax = a; }
    const float dd = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
    int sum[2] = {0, 0};
    for (int i = 0; i < 32; ++i) {
      const int qi = (int)lrintf(v[blk * 32 + i] * inv);
      const int e = blk * 32 + i;
      q[act_chunk_off(e >> 4) + (e & 15)] = (int8_t)qi;
      sum[i >> 4] += qi;
    }
    d[blk] = dd; s16[2 * blk] = sum[0]; s16[2 * blk + 1] = sum[1];
    if (m && (blk >> 1) < k / 64) {
      U4& r = m[blk >> 1];
      if (blk & 1) { r.y = as_u(dd); r.w = (uint32_t)(sum[0] + sum[1]); } else { r.x = as_u(dd); r.z = (uint32_t)(sum[0] + sum[1]); }
    }
  }
}

}  // namespace rlz
