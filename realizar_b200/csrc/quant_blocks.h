// GGML block-quantisation layouts and per-block decoders, shared by the host
// (C++ CPU engine, quantisers) and the device (sm_100a kernels).
//
// Byte layouts are the on-disk GGUF layouts, read unchanged:
//   Q4_0  18 B / 32   : f16 d, 16 B nibbles (low nibble -> elems 0..15, high -> 16..31), y = d*(q-8)
//   Q4_1  20 B / 32   : f16 d, f16 m, 16 B nibbles, y = d*q + m
//   Q5_0  22 B / 32   : f16 d, 4 B high bits, 16 B nibbles, y = d*(q-16)
//   Q5_1  24 B / 32   : f16 d, f16 m, 4 B high bits, 16 B nibbles
//   Q8_0  34 B / 32   : f16 d, 32 x i8
//   Q2_K  84 B / 256  : 16 B scales(4b sc | 4b min), 64 B qs, f16 d, f16 dmin
//   Q4_K 144 B / 256  : f16 d, f16 dmin, 12 B packed 6-bit scales/mins, 128 B nibbles
//   Q5_K 176 B / 256  : f16 d, f16 dmin, 12 B scales, 32 B high bits, 128 B nibbles
//   Q6_K 210 B / 256  : 128 B ql, 64 B qh, 16 x i8 scales, f16 d
// (reference parity: src/quantize/mod.rs:14-56, src/quantize/dequant_q4k.rs,
//  src/cuda/types.rs:99-150).  Q5_K follows the canonical ggml bit order.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define RLZ_HD __host__ __device__ __forceinline__
#include <cuda_fp16.h>
#else
#define RLZ_HD inline
#endif

namespace rlz {

enum QType : int {
  QT_F32 = 0, QT_F16 = 1, QT_Q4_0 = 2, QT_Q4_1 = 3, QT_Q5_0 = 6, QT_Q5_1 = 7,
  QT_Q8_0 = 8, QT_Q8_1 = 9, QT_Q2_K = 10, QT_Q3_K = 11, QT_Q4_K = 12, QT_Q5_K = 13,
  QT_Q6_K = 14, QT_BF16 = 30,
};

constexpr int QK_K = 256;

// block size in elements / bytes for a ggml type id; 0 if unsupported.
RLZ_HD int qtype_block_elems(int t) {
  switch (t) {
    case QT_F32: case QT_F16: case QT_BF16: return 1;
    case QT_Q4_0: case QT_Q4_1: case QT_Q5_0: case QT_Q5_1: case QT_Q8_0: case QT_Q8_1: return 32;
    case QT_Q2_K: case QT_Q3_K: case QT_Q4_K: case QT_Q5_K: case QT_Q6_K: return 256;
    default: return 0;
  }
}
RLZ_HD int qtype_block_bytes(int t) {
  switch (t) {
    case QT_F32: return 4; case QT_F16: case QT_BF16: return 2;
    case QT_Q4_0: return 18; case QT_Q4_1: return 20; case QT_Q5_0: return 22; case QT_Q5_1: return 24;
    case QT_Q8_0: return 34; case QT_Q8_1: return 36;
    case QT_Q2_K: return 84; case QT_Q3_K: return 110; case QT_Q4_K: return 144;
    case QT_Q5_K: return 176; case QT_Q6_K: return 210;
    default: return 0;
  }
}

// ---- fp16 / bf16 <-> fp32 without relying on hardware types on the host -------------
RLZ_HD float half_bits_to_float(uint16_t h) {
#if defined(__CUDA_ARCH__)
  return __half2float(__ushort_as_half(h));
#else
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) { bits = sign; }
    else {  // subnormal: normalise
      int e = -1;
      do { e++; man <<= 1; } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f; memcpy(&f, &bits, 4); return f;
#endif
}

inline uint16_t float_to_half_bits(float f) {  // round-to-nearest-even, host only
  uint32_t x; memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
  if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);            // overflow -> inf
  if (absx < 0x33000001u) return (uint16_t)sign;                          // underflow -> 0
  int exp = (int)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  if (exp < -14) {  // subnormal half
    int shift = -14 - exp + 13;
    uint32_t r = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (r & 1))) r++;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(exp + 15) << 10) | ((man >> 13) & 0x3FFu);
  uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
  return (uint16_t)(sign | r);
}

RLZ_HD float bf16_bits_to_float(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
#if defined(__CUDA_ARCH__)
  return __uint_as_float(bits);
#else
  float f; memcpy(&f, &bits, 4); return f;
#endif
}
inline uint16_t float_to_bf16_bits(float f) {
  uint32_t x; memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

RLZ_HD uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

// 6-bit scale / min of sub-block j (0..7) from the 12 packed bytes of Q4_K / Q5_K.
RLZ_HD void get_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
  if (j < 4) {
    *sc = q[j] & 63; *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m  = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// ---- per-block decoders: write `block elems` floats to y ------------------------------
RLZ_HD void dequant_block_q4_0(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b));
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; ++j) {
    y[j] = d * (float)((int)(qs[j] & 0xF) - 8);
    y[j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
  }
}
RLZ_HD void dequant_block_q4_1(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b)), m = half_bits_to_float(load_u16(b + 2));
  const uint8_t* qs = b + 4;
  for (int j = 0; j < 16; ++j) {
    y[j] = d * (float)(qs[j] & 0xF) + m;
    y[j + 16] = d * (float)(qs[j] >> 4) + m;
  }
}
RLZ_HD void dequant_block_q5_0(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b));
  uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
  const uint8_t* qs = b + 6;
  for (int j = 0; j < 16; ++j) {
    const int xh0 = (int)((qh >> j) & 1u) << 4;
    const int xh1 = (int)((qh >> (j + 16)) & 1u) << 4;
    y[j] = d * (float)(((qs[j] & 0xF) | xh0) - 16);
    y[j + 16] = d * (float)(((qs[j] >> 4) | xh1) - 16);
  }
}
RLZ_HD void dequant_block_q5_1(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b)), m = half_bits_to_float(load_u16(b + 2));
  uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
  const uint8_t* qs = b + 8;
  for (int j = 0; j < 16; ++j) {
    const int xh0 = (int)((qh >> j) & 1u) << 4;
    const int xh1 = (int)((qh >> (j + 16)) & 1u) << 4;
    y[j] = d * (float)((qs[j] & 0xF) | xh0) + m;
    y[j + 16] = d * (float)((qs[j] >> 4) | xh1) + m;
  }
}
RLZ_HD void dequant_block_q8_0(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b));
  const int8_t* qs = (const int8_t*)(b + 2);
  for (int j = 0; j < 32; ++j) y[j] = d * (float)qs[j];
}
RLZ_HD void dequant_block_q2_k(const uint8_t* b, float* y) {
  const uint8_t* scales = b; const uint8_t* q = b + 16;
  const float d = half_bits_to_float(load_u16(b + 80)), dmin = half_bits_to_float(load_u16(b + 82));
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc = scales[is++];
      float dl = d * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
      for (int l = 0; l < 16; ++l) *y++ = dl * (float)((q[l] >> shift) & 3) - ml;
      sc = scales[is++];
      dl = d * (float)(sc & 0xF); ml = dmin * (float)(sc >> 4);
      for (int l = 0; l < 16; ++l) *y++ = dl * (float)((q[l + 16] >> shift) & 3) - ml;
      shift += 2;
    }
    q += 32;
  }
}
RLZ_HD void dequant_block_q4_k(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b)), dmin = half_bits_to_float(load_u16(b + 2));
  const uint8_t* scales = b + 4; const uint8_t* q = b + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    get_scale_min_k4(is + 0, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = dmin * (float)m;
    get_scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * (float)(q[l] & 0xF) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * (float)(q[l] >> 4) - m2;
    q += 32; is += 2;
  }
}
RLZ_HD void dequant_block_q5_k(const uint8_t* b, float* y) {
  const float d = half_bits_to_float(load_u16(b)), dmin = half_bits_to_float(load_u16(b + 2));
  const uint8_t* scales = b + 4; const uint8_t* qh = b + 16; const uint8_t* ql = b + 48;
  int is = 0; uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    get_scale_min_k4(is + 0, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = dmin * (float)m;
    get_scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32; is += 2; u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
  }
}
RLZ_HD void dequant_block_q6_k(const uint8_t* b, float* y) {
  const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192);
  const float d = half_bits_to_float(load_u16(b + 208));
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l] = d * (float)sc[is + 0] * (float)q1;
      y[l + 32] = d * (float)sc[is + 2] * (float)q2;
      y[l + 64] = d * (float)sc[is + 4] * (float)q3;
      y[l + 96] = d * (float)sc[is + 6] * (float)q4;
    }
    y += 128; ql += 64; qh += 32; sc += 8;
  }
}

// Decode one block of any supported block type.  Returns false for unsupported types.
RLZ_HD bool dequant_block(int qtype, const uint8_t* b, float* y) {
  switch (qtype) {
    case QT_Q4_0: dequant_block_q4_0(b, y); return true;
    case QT_Q4_1: dequant_block_q4_1(b, y); return true;
    case QT_Q5_0: dequant_block_q5_0(b, y); return true;
    case QT_Q5_1: dequant_block_q5_1(b, y); return true;
    case QT_Q8_0: dequant_block_q8_0(b, y); return true;
    case QT_Q2_K: dequant_block_q2_k(b, y); return true;
    case QT_Q4_K: dequant_block_q4_k(b, y); return true;
    case QT_Q5_K: dequant_block_q5_k(b, y); return true;
    case QT_Q6_K: dequant_block_q6_k(b, y); return true;
    default: return false;
  }
}

}  // namespace rlz
