// The decode GEMV as a device function: input staging (fused norm + int8 quantisation), the row loops and the
// epilogue.  Used by the one-launch-per-GEMV kernel and by the persistent decode-step kernel.
#pragma once
#include "common.cuh"
#include "../gemv_units.h"
#include "gemv_params.h"
#include "gemv_common.cuh"

namespace rlz {

constexpr int GEMV_THREADS = 512;
#ifndef GEMV_OCC2_MAXB
#define GEMV_OCC2_MAXB 1          // batch sizes up to this run two CTAs per SM (64 registers per thread)
#endif
#ifndef GEMV_UNROLL
#define GEMV_UNROLL 1          // rolled unit loop: smaller code measured faster at decode sizes
#endif
#ifndef GEMV_RG_ROWS
#define GEMV_RG_ROWS 4
#endif
#ifndef GEMV_REG_STAGING
#define GEMV_REG_STAGING 0        // 1: stage the input through registers (larger code, one memory round trip)
#endif

// int8 staging in the ActView layout: xq[B][k] (chunk-rotated), xd[B][k/32], xs[B][k/16] (int sums),
// xm[B][k/64] records {d0, d1, sum32_0, sum32_1}
template <int B>
__device__ void stage_x_q8(const GemvX& X, int8_t* xq, float* xd, int32_t* xs, uint32_t* xm, float* red) {
  const int k = X.k;
#pragma unroll 1
  for (int b = 0; b < B; ++b) {
    const float* x = X.x + (int64_t)b * X.ld;
    float mean, rstd;
    row_stats(X, x, red, &mean, &rstd);
    // groups of 8 lanes own one 32-block; the loop bound is warp-uniform so shuffles are safe
    for (int base = (threadIdx.x & ~31) * 4; base < k; base += blockDim.x * 4) {
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
        *(uint32_t*)(xq + (int64_t)b * k + act_chunk_off(i >> 4) + (i & 15)) =
            (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
        if ((threadIdx.x & 3) == 0) xs[(int64_t)b * (k >> 4) + (i >> 4)] = s16;
        if ((threadIdx.x & 7) == 0) {
          xd[(int64_t)b * (k >> 5) + (i >> 5)] = d;
          uint32_t* rec = xm + ((int64_t)b * (k >> 6) + (i >> 6)) * 4 + ((i >> 5) & 1);
          rec[0] = __float_as_uint(d);
          rec[2] = (uint32_t)s32;
        }
      }
    }
  }
}

// f32 staging for dense / generic block types: xf[B][k]
template <int B>
__device__ void stage_x_f32(const GemvX& X, float* xf, float* red) {
#pragma unroll 1
  for (int b = 0; b < B; ++b) {
    const float* x = X.x + (int64_t)b * X.ld;
    float mean, rstd;
    row_stats(X, x, red, &mean, &rstd);
    for (int i = threadIdx.x * 4; i < X.k; i += blockDim.x * 4)
      *(float4*)(xf + (int64_t)b * X.k + i) = load_normed(X, x, i, mean, rstd);
  }
}

// ---- row loops ---------------------------------------------------------------------------
// A warp takes GEMV_RG consecutive rows at a time and its lanes stride over the flattened
// (row, unit) space of that group, so every lane has several independent 16-byte weight loads
// in flight even when a single row is only a few units long.
constexpr int GEMV_RG = GEMV_RG_ROWS;
constexpr int GEMV_UNROLL_C = GEMV_UNROLL;

template <int QT, int B>
__device__ __forceinline__ void rows_q8(const GemvSeg& S, int r0, int r1, const ActView& a, float* rowacc, float* part, int s) {
  const int upr = dev_units_per_row(QT, S.k);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int ngroups = (r1 - r0 + GEMV_RG - 1) / GEMV_RG;
  // few rows per CTA: several warps share one row group (each takes every `share`-th slice of
  // 32 units) and their partial sums are combined through shared memory in a fixed order
  const int share = ngroups >= nw || ngroups == 0 ? 1 : nw / ngroups;
  const int gstep = share == 1 ? nw : ngroups;           // share > 1: every group is visited once
  const int sub = share == 1 ? 0 : warp % share;
  for (int gi = share == 1 ? warp : warp / share; gi < ngroups; gi += gstep) {
    const int g0 = r0 + gi * GEMV_RG;
    const int rows = min(GEMV_RG, r1 - g0);
    const uint8_t* base = S.W + (int64_t)g0 * S.stride;
    const int total = rows * upr;
    float acc[GEMV_RG][B];
#pragma unroll
    for (int r = 0; r < GEMV_RG; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    int rl = 0, u = sub * 32 + lane;            // row within the group, unit within the row
    while (u >= upr) { u -= upr; ++rl; }
    const int fstep = 32 * share;
#pragma unroll GEMV_UNROLL_C
    for (int f = sub * 32 + lane; f < total; f += fstep) {
      float t[B];
#pragma unroll
      for (int b = 0; b < B; ++b) t[b] = 0.f;
      unit_dot<QT, B>(base + (int64_t)rl * S.stride, u, a, t);
#pragma unroll
      for (int r = 0; r < GEMV_RG; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] += rl == r ? t[b] : 0.f;
      u += fstep;
      while (u >= upr) { u -= upr; ++rl; }
    }
#pragma unroll
    for (int r = 0; r < GEMV_RG; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = warp_sum(acc[r][b]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < GEMV_RG; ++r) {
#pragma unroll
        for (int b = 0; b < B; ++b) {
          if (share == 1) { if (r < rows) rowacc[((g0 + r - r0) * 2 + s) * B + b] = acc[r][b]; }
          else part[(warp * GEMV_RG + r) * B + b] = acc[r][b];
        }
      }
    }
    if (share > 1) break;                       // one group per warp in the shared regime
  }
  if (share > 1) {                              // uniform over the CTA
    __syncthreads();
    for (int idx = threadIdx.x; idx < (r1 - r0) * B; idx += blockDim.x) {
      const int rl = idx / B, b = idx - rl * B, gi = rl / GEMV_RG, r = rl - gi * GEMV_RG;
      float v = 0.f;
      for (int w = 0; w < share; ++w) v += part[((gi * share + w) * GEMV_RG + r) * B + b];
      rowacc[(rl * 2 + s) * B + b] = v;
    }
    __syncthreads();
  }
}

// generic path: any block type through the plain block decoders, f32 activations
template <int B>
__device__ void rows_f32(const GemvSeg& S, int r0, int r1, const float* xf, float* rowacc, int s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int be = qtype_block_elems(S.qtype), bb = qtype_block_bytes(S.qtype);
  for (int r = r0 + warp; r < r1; r += nw) {
    const uint8_t* row = S.W + (int64_t)r * S.stride;
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.f;
    if (be == 1) {   // dense rows: 4 elements per lane step
      for (int i = lane * 4; i < S.k; i += 128) {
        float w[4];
        if (S.qtype == QT_F32) { const float4 t = *(const float4*)(row + (int64_t)i * 4); w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w; }
        else {
          const uint2 t = *(const uint2*)(row + (int64_t)i * 2);
          const uint32_t h[4] = {t.x & 0xFFFFu, t.x >> 16, t.y & 0xFFFFu, t.y >> 16};
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = S.qtype == QT_F16 ? h2f(h[j]) : __uint_as_float(h[j] << 16);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const float4 xv = *(const float4*)(xf + (int64_t)b * S.k + i);
          acc[b] += w[0] * xv.x + w[1] * xv.y + w[2] * xv.z + w[3] * xv.w;
        }
      }
    } else {
      const int nblk = S.k / be;
      for (int blk = lane; blk < nblk; blk += 32) {
        float tmp[256];
        dequant_block(S.qtype, row + (int64_t)blk * bb, tmp);
        for (int b = 0; b < B; ++b) {
          const float* xb = xf + (int64_t)b * S.k + (int64_t)blk * be;
          float t = 0.f;
          for (int j = 0; j < be; ++j) t += tmp[j] * xb[j];
          acc[b] += t;
        }
      }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = warp_sum(acc[b]);
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < B; ++b) rowacc[((r - r0) * 2 + s) * B + b] = acc[b];
    }
  }
}

// Optional phase trace of the standalone kernel (diagnostics): thread 0 of every CTA records the global timer at
// entry, after the dependency wait, after input staging, after the row loops and after the epilogue.
constexpr int GEMV_TRACE_CTAS = 512, GEMV_TRACE_PTS = 8;
static __device__ int g_gemv_trace_on = 0;
static __device__ unsigned long long g_gemv_trace[GEMV_TRACE_CTAS * GEMV_TRACE_PTS];
__device__ __forceinline__ void gemv_trace(bool on, int cta, int pt) {
  if (on) {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_gemv_trace[cta * GEMV_TRACE_PTS + pt] = t;
  }
}

// L2 prefetch of the weight slab that CTA `bx` of the launch described by p will read
__device__ __forceinline__ void gemv_prefetch_slab(const GemvParams& p, int bx) {
  int m = 0;
  while (m + 1 < p.nmat && bx >= p.mat[m + 1].cta_begin) ++m;
  const GemvMat& M = p.mat[m];
  const int r0 = (bx - M.cta_begin) * M.rows_per_cta;
  const int r1 = min(M.n, r0 + M.rows_per_cta);
  for (int s = 0; s < M.nseg; ++s) {
    const uint8_t* base = M.seg[s].W + (int64_t)r0 * M.seg[s].stride;
    const int64_t bytes = (int64_t)max(0, r1 - r0) * M.seg[s].stride;
    for (int64_t off = (int64_t)threadIdx.x * 128; off < bytes; off += (int64_t)blockDim.x * 128) prefetch_l2(base + off);
  }
}

// The work of CTA `bx` of a GEMV launch.  STANDALONE: one kernel launch per GEMV (weight prefetch ahead of the programmatic
// dependency wait); otherwise the caller is a persistent kernel that has prefetched already and orders launches itself.
template <int B, bool FAST, bool STANDALONE>
__device__ __forceinline__ void gemv_body(const GemvParams& p, const int bx, uint8_t* smem) {
  int m = 0;
  while (m + 1 < p.nmat && bx >= p.mat[m + 1].cta_begin) ++m;
  const GemvMat& M = p.mat[m];
  const int r0 = (bx - M.cta_begin) * M.rows_per_cta;
  const int r1 = min(M.n, r0 + M.rows_per_cta);

  const bool tr = STANDALONE && threadIdx.x == 0 && bx < GEMV_TRACE_CTAS && g_gemv_trace_on;
  gemv_trace(tr, bx, 0);
  if (STANDALONE) {
    gemv_prefetch_slab(p, bx);                    // pull this CTA's weight slab towards L2 while the previous kernel drains
    pdl_launch_dependents();
    pdl_wait();
  }
  gemv_trace(tr, bx, 1);

  // shared memory carve-up (sizes fixed by the launcher from max_k / max_rows)
  const int kq = p.max_k;
  constexpr bool fast = FAST;
  int8_t* xq = (int8_t*)smem;
  uint32_t* xm = (uint32_t*)(smem + (size_t)B * kq);
  float* xd = (float*)(xm + (size_t)B * (kq >> 6) * 4);
  int32_t* xs = (int32_t*)(xd + (size_t)B * (kq >> 5));
  float* xf = (float*)smem;
  const size_t act_bytes = !FAST ? (size_t)B * kq * 4 : (size_t)B * kq + (size_t)B * (kq >> 6) * 16 + (size_t)B * (kq >> 5) * 4 + (size_t)B * (kq >> 4) * 4;
  float* red = (float*)(smem + ((act_bytes + 15) & ~(size_t)15));
  float* part = red + 40;                                  // [warps][GEMV_RG][B] partial sums
  float* rowacc = part + (GEMV_THREADS / 32) * GEMV_RG * B;

  int staged = -1;
  for (int s = 0; s < M.nseg; ++s) {
    const GemvSeg& S = M.seg[s];
    if (S.x_id != staged) {
      __syncthreads();
      const GemvX& X = p.xs[S.x_id];
      const bool in_regs = GEMV_REG_STAGING && X.k <= STAGE_MAXV * 4 * GEMV_THREADS;
      if constexpr (fast) {
        if (B == 1 && X.pre) {                              // the producer left this activation quantised: plain 16-byte copies
          const int k = X.k;                                // sections of the block: codes | per-64 records | per-32 scales | per-16 sums
          const uint8_t* g = X.pre;
          const int n_q = k >> 4, n_m = k >> 6, n_d = k >> 7, n_s = k >> 6;      // 16-byte vectors per section (k is a multiple of 128)
          for (int i = threadIdx.x; i < n_q; i += blockDim.x) ((uint4*)xq)[i] = ((const uint4*)g)[i];
          for (int i = threadIdx.x; i < n_m; i += blockDim.x) ((uint4*)xm)[i] = ((const uint4*)(g + k))[i];
          for (int i = threadIdx.x; i < n_d; i += blockDim.x) ((uint4*)xd)[i] = ((const uint4*)(g + k + (k >> 2)))[i];
          for (int i = threadIdx.x; i < n_s; i += blockDim.x) ((uint4*)xs)[i] = ((const uint4*)(g + k + (k >> 2) + (k >> 3)))[i];
        } else if (in_regs) {
          const int k = X.k;
          stage_rows_regs<B, true>(X, red,
            [&](int b, int i, uint32_t packed, float d, int s16, int s32) {
              *(uint32_t*)(xq + (int64_t)b * k + act_chunk_off(i >> 4) + (i & 15)) = packed;
              if ((threadIdx.x & 3) == 0) xs[(int64_t)b * (k >> 4) + (i >> 4)] = s16;
              if ((threadIdx.x & 7) == 0) {
                xd[(int64_t)b * (k >> 5) + (i >> 5)] = d;
                uint32_t* rec = xm + ((int64_t)b * (k >> 6) + (i >> 6)) * 4 + ((i >> 5) & 1);
                rec[0] = __float_as_uint(d); rec[2] = (uint32_t)s32;
              }
            },
            [](int, int, float4) {});
        } else stage_x_q8<B>(X, xq, xd, xs, xm, red);
      } else {
        if (in_regs) {
          const int k = X.k;
          stage_rows_regs<B, false>(X, red, [](int, int, uint32_t, float, int, int) {},
                                    [&](int b, int i, float4 w) { *(float4*)(xf + (int64_t)b * k + i) = w; });
        } else stage_x_f32<B>(X, xf, red);
      }
      staged = S.x_id;
      __syncthreads();
      gemv_trace(tr, bx, 2 + (s > 0 ? 2 : 0));    // 2: first input staged; 4: second input staged
    }
    if constexpr (fast) {
      const ActView a{xq, xd, xs, (const U4*)xm, S.k};
      switch (S.qtype) {
        case QT_Q4_K: rows_q8<QT_Q4_K, B>(S, r0, r1, a, rowacc, part, s); break;
        case QT_Q5_K: rows_q8<QT_Q5_K, B>(S, r0, r1, a, rowacc, part, s); break;
        case QT_Q6_K: rows_q8<QT_Q6_K, B>(S, r0, r1, a, rowacc, part, s); break;
#ifndef GEMV_ONLY_KQ
        case QT_Q8_0: rows_q8<QT_Q8_0, B>(S, r0, r1, a, rowacc, part, s); break;
        default: rows_q8<QT_Q4_0, B>(S, r0, r1, a, rowacc, part, s); break;
#else
        default: break;
#endif
      }
    } else {
      rows_f32<B>(S, r0, r1, xf, rowacc, s);
    }
    gemv_trace(tr, bx, 3 + (s > 0 ? 2 : 0));      // 3: rows of the first segment done; 5: of the second
  }
  __syncthreads();
  gemv_trace(tr, bx, 6);

  gemv_epilogue<B>(p, M, rowacc, r0, r1);
  gemv_trace(tr, bx, 7);
}

inline size_t gemv_smem_bytes(const GemvParams& p) {
  const size_t B = (size_t)p.batch, kq = (size_t)p.max_k;
  const size_t act = p.any_generic ? B * kq * 4 : B * kq + B * (kq >> 6) * 16 + B * (kq >> 5) * 4 + B * (kq >> 4) * 4;
  return ((act + 15) & ~(size_t)15) + 40 * 4 + (size_t)(GEMV_THREADS / 32) * GEMV_RG * B * 4 + (size_t)p.max_rows * 2 * B * 4;
}

// Validate a launch description and fill in the derived fields (first CTA of each matrix, staging sizes).
// Returns 0 or a negative code; *grid_out receives the number of CTAs.
inline int gemv_prepare(GemvParams& p, int* grid_out) {
  if (p.nmat < 1 || p.nmat > GEMV_MAX_MATS || p.batch < 1 || p.batch > 4) return -1;
  if (p.ar.enabled && (p.nmat != 1 || p.ar.world < 1 || p.ar.world > GEMV_AR_MAX_RANKS || p.mat[0].out_off != 0)) return -8;
  int grid = 0, max_rows = 0, max_k = 0, any_generic = 0;
  for (int m = 0; m < p.nmat; ++m) {
    GemvMat& M = p.mat[m];
    if (M.nseg < 1 || M.nseg > 2 || M.n < 1 || M.rows_per_cta < 1) return -2;
    if (M.q_out && (p.batch != 1 || M.rows_per_cta % 32 || M.q_out_col0 % 32 || M.q_out_k % 128 || M.q_out_col0 + M.n > M.q_out_k || ((uintptr_t)M.q_out & 15))) return -9;
    const bool fast0 = M.seg[0].qtype == QT_Q4_K || M.seg[0].qtype == QT_Q5_K || M.seg[0].qtype == QT_Q6_K || M.seg[0].qtype == QT_Q8_0 || M.seg[0].qtype == QT_Q4_0;
    for (int s = 0; s < M.nseg; ++s) {
      const GemvSeg& S = M.seg[s];
      const bool f = S.qtype == QT_Q4_K || S.qtype == QT_Q5_K || S.qtype == QT_Q6_K || S.qtype == QT_Q8_0 || S.qtype == QT_Q4_0;
      if (f != fast0) return -3;                        // a matrix is all fast-path or all generic
      if (!f) any_generic = 1;
      if (m > 0 && (int)!f != any_generic) return -3;   // and so is a launch
      if (S.x_id < 0 || S.x_id >= GEMV_MAX_X || p.xs[S.x_id].k != S.k) return -4;
      if (S.k % 32 || (f && S.k % 64) || (S.stride & 15) || ((uintptr_t)S.W & 15)) return -5;   // int8 path stages 64-value groups
      if (qtype_block_elems(S.qtype) == 0 || S.k % qtype_block_elems(S.qtype)) return -6;
      if (S.k > max_k) max_k = S.k;
    }
    M.cta_begin = grid;
    grid += (M.n + M.rows_per_cta - 1) / M.rows_per_cta;
    if (M.rows_per_cta > max_rows) max_rows = M.rows_per_cta;
  }
  p.max_k = max_k; p.max_rows = max_rows; p.any_generic = any_generic;
  if (gemv_smem_bytes(p) > 226 * 1024) return -7;
  if (p.ar.enabled && p.mat[0].n > p.ar.n) return -9;
  *grid_out = grid;
  return 0;
}


}  // namespace rlz
