// Pieces shared by the decode GEMV kernels: fused-norm statistics and normalised loads of the
// input vector, and the common epilogue.
#pragma once
#include "common.cuh"
#include "gemv_params.h"

namespace rlz {

// ---- input staging ---------------------------------------------------------------------
// mean / rstd of one input row (block-wide).  LayerNorm uses two passes for accuracy.
__device__ inline void row_stats(const GemvX& X, const float* x, float* red, float* mean_out, float* rstd_out) {
  float mean = 0.f, rstd = 1.f;
  if (X.norm == NORM_RMS) {
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < X.k; i += blockDim.x * 4) {
      const float4 v = *(const float4*)(x + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)X.k + X.eps);
  } else if (X.norm == NORM_LAYER) {
    float s = 0.f;
    for (int i = threadIdx.x * 4; i < X.k; i += blockDim.x * 4) {
      const float4 v = *(const float4*)(x + i);
      s += v.x + v.y + v.z + v.w;
    }
    mean = block_sum(s, red) / (float)X.k;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < X.k; i += blockDim.x * 4) {
      const float4 v = *(const float4*)(x + i);
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      ss += a * a + b * b + c * c + d * d;
    }
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)X.k + X.eps);
  }
  *mean_out = mean; *rstd_out = rstd;
}

__device__ __forceinline__ float4 load_normed(const GemvX& X, const float* x, int i, float mean, float rstd) {
  float4 v = *(const float4*)(x + i);
  if (X.norm != NORM_NONE) {
    v.x = (v.x - mean) * rstd; v.y = (v.y - mean) * rstd; v.z = (v.z - mean) * rstd; v.w = (v.w - mean) * rstd;
    if (X.nw) { const float4 w = __ldg((const float4*)(X.nw + i)); v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w; }
    if (X.nb) { const float4 b = __ldg((const float4*)(X.nb + i)); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
  }
  return v;
}


// ---- register-resident staging ---------------------------------------------------------------
// The whole input row is loaded into registers with one batch of independent loads (one memory
// round trip instead of one per loop iteration), the norm statistics are reduced from registers,
// and the normalised values are either quantised to int8 per 32-block (QUANT) or handed over as
// floats.  `sink_q(b, i, packed4, d, s16, s32)` receives four consecutive int8 values starting at
// element i, the scale of their 32-block and the integer sums of their 16- and 32-element groups
// (valid in every lane of the group); `sink_f(b, i, v)` receives four floats.
// Covers k <= STAGE_MAXV * 4 * blockDim.x; callers fall back to the looped staging beyond that.
constexpr int STAGE_MAXV = 16;

template <int B, bool QUANT, class SinkQ, class SinkF>
__device__ __forceinline__ void stage_rows_regs(const GemvX& X, float* red, SinkQ&& sink_q, SinkF&& sink_f) {
  const int k = X.k, nt = blockDim.x, tid = threadIdx.x;
#pragma unroll 1
  for (int b = 0; b < B; ++b) {
    const float* x = X.x + (int64_t)b * X.ld;
    float4 v[STAGE_MAXV];
#pragma unroll
    for (int it = 0; it < STAGE_MAXV; ++it) {
      const int i = (it * nt + tid) * 4;
      v[it] = i < k ? *(const float4*)(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float mean = 0.f, rstd = 1.f;
    if (X.norm != NORM_NONE) {
      float s = 0.f;
      if (X.norm == NORM_LAYER) {
#pragma unroll
        for (int it = 0; it < STAGE_MAXV; ++it) s += v[it].x + v[it].y + v[it].z + v[it].w;     // padding is zero
        mean = block_sum(s, red) / (float)k;
      }
      float ss = 0.f;
#pragma unroll
      for (int it = 0; it < STAGE_MAXV; ++it) {
        if ((it * nt + tid) * 4 < k) {
          const float a = v[it].x - mean, c = v[it].y - mean, d = v[it].z - mean, e = v[it].w - mean;
          ss += a * a + c * c + d * d + e * e;
        }
      }
      ss = block_sum(ss, red);
      rstd = rsqrtf(ss / (float)k + X.eps);
    }
#pragma unroll
    for (int it = 0; it < STAGE_MAXV; ++it) {
      const int i = (it * nt + tid) * 4;
      if (it * nt * 4 >= k) break;                        // uniform over the CTA
      const bool ok = i < k;
      float4 w = v[it];
      if (X.norm != NORM_NONE && ok) {
        w.x = (w.x - mean) * rstd; w.y = (w.y - mean) * rstd; w.z = (w.z - mean) * rstd; w.w = (w.w - mean) * rstd;
        if (X.nw) { const float4 g = __ldg((const float4*)(X.nw + i)); w.x *= g.x; w.y *= g.y; w.z *= g.z; w.w *= g.w; }
        if (X.nb) { const float4 g = __ldg((const float4*)(X.nb + i)); w.x += g.x; w.y += g.y; w.z += g.z; w.w += g.w; }
      }
      if (!QUANT) { if (ok) sink_f(b, i, w); continue; }
      float amax = fmaxf(fmaxf(fabsf(w.x), fabsf(w.y)), fmaxf(fabsf(w.z), fabsf(w.w)));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float d = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
      const int q0 = __float2int_rn(w.x * inv), q1 = __float2int_rn(w.y * inv), q2 = __float2int_rn(w.z * inv), q3 = __float2int_rn(w.w * inv);
      int s16 = q0 + q1 + q2 + q3;
      s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
      s16 += __shfl_xor_sync(0xffffffffu, s16, 2);
      const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 4);
      if (ok) sink_q(b, i, (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24), d, s16, s32);
    }
  }
}

// Value of output (row rl, batch b) before the residual: combine of the segment sums, biases, activation.
template <int B>
__device__ __forceinline__ float gemv_value(const GemvMat& M, const float* rowacc, int rl, int b, int r) {
  float v = rowacc[(rl * 2 + 0) * B + b];
  if (M.nseg == 2) {
    const float v1 = rowacc[(rl * 2 + 1) * B + b];
    if (M.combine == COMBINE_ADD) v += v1;
    else {
      if (M.bias) v += M.bias[r];
      if (M.bias2) { const float u = v1 + M.bias2[r]; v = (M.combine == COMBINE_SILU_MUL ? silu(v) : gelu_tanh(v)) * u; }
      else v = (M.combine == COMBINE_SILU_MUL ? silu(v) : gelu_tanh(v)) * v1;
    }
  }
  if (M.nseg == 1 || M.combine == COMBINE_ADD) {
    if (M.bias) v += M.bias[r];
    if (M.bias2) v += M.bias2[r];
  }
  if (M.act == ACT_GELU) v = gelu_tanh(v); else if (M.act == ACT_SILU) v = silu(v);
  return v;
}

// Epilogue over the rows [r0, r1) of matrix M: rowacc holds [row][segment][batch] sums.
// With p.ar.enabled the partial outputs are all-reduced across the tensor-parallel ranks inside
// the kernel before the residual is added; every rank ends with the same sum.
template <int B>
__device__ __forceinline__ void gemv_epilogue(const GemvParams& p, const GemvMat& M, float* rowacc, int r0, int r1) {
  const int count = (r1 - r0) * B;
  if (!p.ar.enabled) {
    if (B == 1 && M.q_out) {
      // a warp owns 32 consecutive outputs = one quantisation block of the next launch's activation (r0 is a multiple of 32)
      const int k = M.q_out_k, lane = threadIdx.x & 31;
      uint8_t* q = M.q_out;
      uint32_t* xm = (uint32_t*)(q + k);
      float* xd = (float*)(xm + (size_t)(k >> 6) * 4);
      int32_t* xs = (int32_t*)(xd + (k >> 5));
      for (int base = (threadIdx.x & ~31); base < count; base += blockDim.x) {
        const int rl = base + lane, r = r0 + rl;
        const bool ok = rl < count;
        float v = ok ? gemv_value<1>(M, rowacc, rl, 0, r) : 0.f;
        if (ok && M.has_residual) v += p.residual[r];
        if (ok) p.y[M.out_off + r] = v;
        const float amax = warp_max(fabsf(v));
        const float d = amax / 127.f, inv = amax > 0.f ? 127.f / amax : 0.f;
        const int qi = __float2int_rn(v * inv);
        int s16 = qi;
        s16 += __shfl_xor_sync(0xffffffffu, s16, 1); s16 += __shfl_xor_sync(0xffffffffu, s16, 2);
        s16 += __shfl_xor_sync(0xffffffffu, s16, 4); s16 += __shfl_xor_sync(0xffffffffu, s16, 8);
        const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 16);
        const int i = M.q_out_col0 + r;                   // position in the destination activation
        if (ok) q[act_chunk_off(i >> 4) + (i & 15)] = (uint8_t)(qi & 0xFF);
        if ((lane & 15) == 0 && ok) xs[i >> 4] = s16;
        if (lane == 0 && ok) {
          xd[i >> 5] = d;
          uint32_t* rec = xm + (size_t)(i >> 6) * 4 + ((i >> 5) & 1);
          rec[0] = __float_as_uint(d);
          rec[2] = (uint32_t)s32;
        }
      }
      return;
    }
    for (int idx = threadIdx.x; idx < count; idx += blockDim.x) {
      const int rl = idx / B, b = idx - rl * B, r = r0 + rl;
      float v = gemv_value<B>(M, rowacc, rl, b, r);
      if (M.has_residual) v += p.residual[(int64_t)b * p.ld_res + r];
      p.y[(int64_t)b * p.ldy + M.out_off + r] = v;
    }
    return;
  }
  const GemvAr& ar = p.ar;
  const uint32_t epoch = *ar.epoch;
  const int64_t slot = (int64_t)ar.n * 4;                        // pairs per (parity, rank) slot
  const int64_t base = (int64_t)(epoch & 1u) * ar.world * slot;
  const int world = ar.world;
  if ((world & (world - 1)) == 0) {
    // One thread per (output, peer) pair: a CTA owns only a handful of rows, so this puts rows x world independent remote
    // stores and polls in flight instead of `world` serial ones per row.  The partial values first go to slot 0 of their
    // rows in shared memory (every thread reads only its own element there).
    for (int idx = threadIdx.x; idx < count; idx += blockDim.x) {
      const int rl = idx / B, b = idx - rl * B;
      const float v = gemv_value<B>(M, rowacc, rl, b, r0 + rl);
      rowacc[(rl * 2) * B + b] = v;
    }
    __syncthreads();
    const int total = count * world, lane = threadIdx.x & 31;
    for (int first = threadIdx.x & ~31; first < total; first += blockDim.x) {      // warp-uniform bound: the shuffles below are safe
      const int idx = first + lane;
      const bool ok = idx < total;
      const int e = ok ? idx / world : 0, q = idx & (world - 1);
      const int rl = e / B, b = e - rl * B, r = r0 + rl;
      const int64_t off = (int64_t)b * ar.n + r;
      float v = 0.f;
      if (ok) {
        // 1. my partial value, tagged with the epoch, into my slot of rank q's inbox
        st_pair_sys(ar.inbox[q] + base + (int64_t)ar.rank * slot + off, __float_as_uint(rowacc[(rl * 2) * B + b]), epoch);
        // 2. rank q's partial value of the same element from my inbox (bounded polls)
        const uint2* src = ar.inbox[ar.rank] + base + (int64_t)q * slot + off;
        uint2 w = ld_pair_sys(src);
        for (int64_t spins = 0; w.y != epoch; ++spins) {
          if (spins > ar.spin_limit) { atomicExch(ar.status, 2001); break; }
          w = ld_pair_sys(src);
        }
        v = __uint_as_float(w.x);
      }
      // the world values of an element sit in adjacent lanes: a fixed xor tree, identical on every rank
      for (int o = 1; o < world; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (ok && q == 0) {
        if (M.has_residual) v += p.residual[(int64_t)b * p.ld_res + r];
        p.y[(int64_t)b * p.ldy + M.out_off + r] = v;
      }
    }
    return;
  }
  for (int idx = threadIdx.x; idx < count; idx += blockDim.x) {
    const int rl = idx / B, b = idx - rl * B, r = r0 + rl;
    // 1. push my partial value, tagged with the epoch, into my slot of every rank's inbox
    const uint32_t bits = __float_as_uint(gemv_value<B>(M, rowacc, rl, b, r));
    const int64_t off = (int64_t)b * ar.n + r;
    for (int q = 0; q < ar.world; ++q) st_pair_sys(ar.inbox[q] + base + (int64_t)ar.rank * slot + off, bits, epoch);
    // 2. collect the same element from every rank's slot of my inbox (bounded polls), sum in rank order
    float v = 0.f;
    for (int q = 0; q < ar.world; ++q) {
      const uint2* src = ar.inbox[ar.rank] + base + (int64_t)q * slot + off;
      uint2 w = ld_pair_sys(src);
      for (int64_t spins = 0; w.y != epoch; ++spins) {
        if (spins > ar.spin_limit) { atomicExch(ar.status, 2001); break; }
        w = ld_pair_sys(src);
      }
      v += __uint_as_float(w.x);
    }
    if (M.has_residual) v += p.residual[(int64_t)b * p.ld_res + r];
    p.y[(int64_t)b * p.ldy + M.out_off + r] = v;
  }
}

}  // namespace rlz
