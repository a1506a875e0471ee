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
    case QT_Q4_K: case QT_Q5_K: return k / 32;
    case QT_Q6_K: return k / 64;
    case QT_Q8_0: return k / 16;
    case QT_Q4_0: return k / 32;
    default: return 0;
  }
}

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ U4 ld_w16(const uint8_t* p) {   // streaming weight load: read once
  U4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
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

struct ActView {         // activations of B rows, row strides derived from k
  const int8_t* q; const float* d; const float* s; int k;
};

// ---- Q4_K: unit u covers sub-blocks (2g, 2g+1) elements [16h, 16h+16) ---------------------
template <int B>
RLZ_HD void unit_q4k(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int sb = u >> 3, t = u & 7, g = t >> 1, h = t & 1;
  const uint8_t* base = row + (int64_t)sb * 144;
  const U4 hdr = ld_c16(base);
  const U4 qs = ld_w16(base + 16 + 16 * t);
  const float d = h2f(hdr.x & 0xFFFFu), dmin = h2f(hdr.x >> 16);
  float sc0, m0, sc1, m1;
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g, &sc0, &m0);
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g + 1, &sc1, &m1);
  const U4 lo{qs.x & 0x0F0F0F0Fu, qs.y & 0x0F0F0F0Fu, qs.z & 0x0F0F0F0Fu, qs.w & 0x0F0F0F0Fu};
  const U4 hi{(qs.x >> 4) & 0x0F0F0F0Fu, (qs.y >> 4) & 0x0F0F0F0Fu, (qs.z >> 4) & 0x0F0F0F0Fu, (qs.w >> 4) & 0x0F0F0F0Fu};
  const int kb = sb * 256 + g * 64 + h * 16;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const float* xd = a.d + (int64_t)b * (a.k >> 5);
    const float* xs = a.s + (int64_t)b * (a.k >> 4);
    const int dlo = dot16(lo, ld_a16(xq + kb)), dhi = dot16(hi, ld_a16(xq + kb + 32));
    acc[b] += d * (sc0 * xd[kb >> 5] * (float)dlo + sc1 * xd[(kb >> 5) + 1] * (float)dhi)
            - dmin * (m0 * xs[kb >> 4] + m1 * xs[(kb >> 4) + 2]);
  }
}

// ---- Q5_K: as Q4_K plus the fifth bit from qh ----------------------------------------------
template <int B>
RLZ_HD void unit_q5k(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int sb = u >> 3, t = u & 7, g = t >> 1, h = t & 1;
  const uint8_t* base = row + (int64_t)sb * 176;
  const U4 hdr = ld_c16(base);
  const U4 qh = ld_c16(base + 16 + 16 * h);
  const U4 qs = ld_w16(base + 48 + 16 * t);
  const float d = h2f(hdr.x & 0xFFFFu), dmin = h2f(hdr.x >> 16);
  float sc0, m0, sc1, m1;
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g, &sc0, &m0);
  k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g + 1, &sc1, &m1);
  const int s0 = 2 * g, s1 = 2 * g + 1;
  const U4 lo{(qs.x & 0x0F0F0F0Fu) | (((qh.x >> s0) & 0x01010101u) << 4), (qs.y & 0x0F0F0F0Fu) | (((qh.y >> s0) & 0x01010101u) << 4),
              (qs.z & 0x0F0F0F0Fu) | (((qh.z >> s0) & 0x01010101u) << 4), (qs.w & 0x0F0F0F0Fu) | (((qh.w >> s0) & 0x01010101u) << 4)};
  const U4 hi{((qs.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> s1) & 0x01010101u) << 4), ((qs.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> s1) & 0x01010101u) << 4),
              ((qs.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> s1) & 0x01010101u) << 4), ((qs.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> s1) & 0x01010101u) << 4)};
  const int kb = sb * 256 + g * 64 + h * 16;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const float* xd = a.d + (int64_t)b * (a.k >> 5);
    const float* xs = a.s + (int64_t)b * (a.k >> 4);
    const int dlo = dot16(lo, ld_a16(xq + kb)), dhi = dot16(hi, ld_a16(xq + kb + 32));
    acc[b] += d * (sc0 * xd[kb >> 5] * (float)dlo + sc1 * xd[(kb >> 5) + 1] * (float)dhi)
            - dmin * (m0 * xs[kb >> 4] + m1 * xs[(kb >> 4) + 2]);
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
  const float d = h2f(tail.x & 0xFFFFu);
  const uint32_t scw0 = n ? scv.z : scv.x, scw1 = n ? scv.w : scv.y;   // 8 scales of this half
  float sc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = lh + 2 * j;                       // 0..7
    const uint32_t wv = idx < 4 ? scw0 : scw1;
    sc[j] = (float)(int)(int8_t)((wv >> (8 * (idx & 3))) & 0xFFu);
  }
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
    const float* xs = a.s + (int64_t)b * (a.k >> 4);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = kb + 32 * j;
      const int dj = dot16(w[j], ld_a16(xq + kk));
      sum += sc[j] * (xd[kk >> 5] * (float)dj - 32.f * xs[kk >> 4]);
    }
    acc[b] += d * sum;
  }
}

// ---- Q8_0 planar: unit u = 16 weights of block u/2 ------------------------------------------
template <int B>
RLZ_HD void unit_q8_0(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int nb = a.k >> 5, blk = u >> 1;
  const float d = h2f((uint32_t)load_u16(row + 2 * blk));
  const U4 w = ld_w16(row + dev_planar_qoff(nb) + 16 * u);
  const int kb = 16 * u;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int dj = dot16(w, ld_a16(a.q + (int64_t)b * a.k + kb));
    acc[b] += d * a.d[(int64_t)b * nb + blk] * (float)dj;
  }
}

// ---- Q4_0 planar: unit u = block u (low nibbles -> elems 0..15, high -> 16..31) -------------
template <int B>
RLZ_HD void unit_q4_0(const uint8_t* row, int u, const ActView& a, float* acc) {
  const int nb = a.k >> 5;
  const float d = h2f((uint32_t)load_u16(row + 2 * u));
  const U4 qs = ld_w16(row + dev_planar_qoff(nb) + 16 * u);
  const U4 lo{qs.x & 0x0F0F0F0Fu, qs.y & 0x0F0F0F0Fu, qs.z & 0x0F0F0F0Fu, qs.w & 0x0F0F0F0Fu};
  const U4 hi{(qs.x >> 4) & 0x0F0F0F0Fu, (qs.y >> 4) & 0x0F0F0F0Fu, (qs.z >> 4) & 0x0F0F0F0Fu, (qs.w >> 4) & 0x0F0F0F0Fu};
  const int kb = 32 * u;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int8_t* xq = a.q + (int64_t)b * a.k;
    const float* xs = a.s + (int64_t)b * (a.k >> 4);
    const int dj = dot16(lo, ld_a16(xq + kb)) + dot16(hi, ld_a16(xq + kb + 16));
    acc[b] += d * (a.d[(int64_t)b * nb + u] * (float)dj - 8.f * (xs[2 * u] + xs[2 * u + 1]));
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

// Activation quantisation of one 32-block (host form; the kernel does the same arithmetic
// cooperatively): q = rint(v * 127/amax), d = amax/127, s16 = d * sum of each 16 ints.
inline void quantize_act_block32(const float* v, int8_t* q, float* d, float* s16) {
  float amax = 0.f;
  for (int i = 0; i < 32; ++i) { float a = v[i] < 0 ? -v[i] : v[i]; if (a > amax) amax = a; }
  const float dd = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
  int s0 = 0, s1 = 0;
  for (int i = 0; i < 32; ++i) {
    const int qi = (int)lrintf(v[i] * inv);
    q[i] = (int8_t)qi; if (i < 16) s0 += qi; else s1 += qi;
  }
  *d = dd; s16[0] = dd * (float)s0; s16[1] = dd * (float)s1;
}

}  // namespace rlz
