// Causal flash attention for prompt chunks on the 5th-generation tensor cores: a block of 128
// consecutive query positions of one sequence x one query head per CTA, keys and values read from
// the paged bf16 KV cache (the chunk's own rows were appended before the launch).
//
// Per 128-key tile:
//   S = Q K^T          tcgen05.mma  M=128 (queries) N=128 (keys)  K=head_dim, accumulator in TMEM
//   softmax            every thread owns one query row (TMEM lane = row): two sweeps of tcgen05.ld
//                      (row max, then exp2 / sum), P written to shared memory as bf16 in the operand layout
//   O_tile = P V       tcgen05.mma  M=128 N=head_dim K=128 (keys); V is transposed into the K-major
//                      operand layout while it is copied from the cache (into the buffer K occupied)
//   O = O * corr + O_tile   in registers (fp32), corr = exp2(m_old - m_new)
// Masking: causal (key <= query), optional sliding window, keys beyond the context, rows beyond the chunk.
// Every mbarrier wait is bounded; on expiry the CTA records error 3101, frees its tensor memory and returns.
//
// Replaces the reference's flash_attention[_causal] / flash_attention_tensor_core[_causal] (WMMA) kernels and the
// cuBLAS strided-batched QK^T + causal_mask_softmax + PV prefill chain
// (src/cuda/executor/layers/cublas_prefill/attention.rs:23-420, src/cuda/executor/head_dim.rs:319-416).
#include "common.cuh"
#include "tcgen05_common.cuh"
#include "attention_decode_body.cuh"
#include <stdlib.h>

namespace rlz {

__device__ int g_prefill_attn_error = 0;

constexpr int FP_THREADS = 128;
constexpr int FP_PAGE = 16;
constexpr int FP_SLAB = 128 * 128;           // one [128 rows x 64 bf16] swizzled slab

struct AttnPrefillParams {
  const float* qkv;            // [T, ld_qkv] fp32, q section already rotated
  float* out;                  // [T, ld_out] fp32, head-major
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int32_t* page_table;   // [max_pages] of this sequence
  int64_t ld_qkv, ld_out;
  int32_t n_heads, n_kv_heads, head_dim, q_off;
  int32_t n_tokens, pos0;      // chunk rows are positions pos0 .. pos0 + n_tokens - 1
  int32_t window, kv_q8;       // kv_q8: int8 cache rows of head_dim + 16 bytes (codes, then the fp32 row scale)
  float scale;
  int32_t out_bf16;            // 1: `out` is bf16 [T, ld_out] (the operand of the output projection GEMM), else fp32
  const int32_t* pos0_ptr;     // when set, the position of row 0 is read from here (a launch captured in a CUDA graph serves any chunk)
};

template <int D>
__global__ void __launch_bounds__(FP_THREADS) attn_prefill_tcgen05_kernel(const __grid_constant__ AttnPrefillParams p) {
  constexpr int NSLAB = (D + 63) / 64;                  // 64-column slabs covering head_dim
  constexpr uint32_t TMEM_COLS = 256;                    // S: columns 0..127, O tile: columns 128..128+D-1
  extern __shared__ __align__(1024) uint8_t fsm[];
  __shared__ __align__(8) uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_base_s;
  uint8_t* sm = (uint8_t*)(((uintptr_t)fsm + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = sm;                                      // NSLAB slabs
  uint8_t* KVs = Qs + NSLAB * FP_SLAB;                   // K tile (NSLAB slabs), then V^T tile (2 slabs of [D rows x 64 keys])
  uint8_t* Ps = KVs + 2 * FP_SLAB;                       // 2 slabs of [128 queries x 64 keys]
  const int tid = threadIdx.x, warp = tid >> 5;
  const int m0 = blockIdx.x * 128, head = blockIdx.y;
  const int kvh = head / (p.n_heads / p.n_kv_heads);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&bar_s)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&bar_o)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t t_lane = (uint32_t)(warp * 32) << 16;   // this warp's TMEM lanes
  pdl_launch_dependents();
  pdl_wait();
  const int pos0 = p.pos0_ptr ? *p.pos0_ptr : p.pos0;

  // ---- Q tile: my row, fp32 -> bf16, swizzled --------------------------------------------------
  const int qrow = m0 + tid;
  const bool qvalid = qrow < p.n_tokens;
  const int qpos = pos0 + qrow;
  {
    const float* src = p.qkv + (int64_t)min(qrow, p.n_tokens - 1) * p.ld_qkv + p.q_off + head * D;
#pragma unroll
    for (int s = 0; s < NSLAB; ++s) {
      uint32_t v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int j = 64 * s + 2 * i;
        v[i] = (j < D && qvalid) ? pack_bf16(src[j], src[j + 1]) : 0u;
      }
      store_row_sw128(Qs + s * FP_SLAB, tid, v);
    }
  }
  const int ctx = pos0 + p.n_tokens;
  const int kend = min(ctx, pos0 + m0 + 128);          // causal: no key beyond the tile's last query
  const int klo = p.window > 0 ? max(0, pos0 + m0 - p.window + 1) / 128 * 128 : 0;
  const float sc = p.scale * 1.4426950408889634f;
  const uint32_t idesc_s = make_idesc_bf16(128, 128), idesc_o = make_idesc_bf16(128, D);
  float o[D];
#pragma unroll
  for (int j = 0; j < D; ++j) o[j] = 0.f;
  float mrow = -INFINITY, lrow = 0.f;
  bool ok = true;
  uint32_t phase = 0;

  for (int k0 = klo; k0 < kend; k0 += 128, phase ^= 1u) {
    // ---- K tile: key k0 + tid ------------------------------------------------------------------
    const int key = k0 + tid;
    const bool kvalid = key < ctx;
    const int64_t crow = ((int64_t)p.page_table[min(key, ctx - 1) / FP_PAGE] * p.n_kv_heads + kvh) * FP_PAGE + (min(key, ctx - 1) % FP_PAGE);
    const int64_t cbase = crow * D;                       // bf16 rows; int8 rows are D + 16 bytes
    const uint8_t* k8 = (const uint8_t*)p.k_cache + crow * (D + 16);
    const uint8_t* v8 = (const uint8_t*)p.v_cache + crow * (D + 16);
    {
      const uint4* src = (const uint4*)(p.k_cache + cbase);
      const float ksc = (p.kv_q8 && kvalid) ? *(const float*)(k8 + D) : 0.f;
#pragma unroll
      for (int s = 0; s < NSLAB; ++s) {
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int j = 64 * s + 8 * c;
          if (p.kv_q8) {                                  // 8 codes -> 8 bf16
            const uint2 cw = (j < D && kvalid) ? __ldg((const uint2*)(k8 + j)) : make_uint2(0, 0);
            const uint32_t w2[2] = {cw.x, cw.y};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float f0 = ksc * (float)(int8_t)(w2[h] & 0xFF), f1 = ksc * (float)(int8_t)((w2[h] >> 8) & 0xFF);
              const float f2 = ksc * (float)(int8_t)((w2[h] >> 16) & 0xFF), f3 = ksc * (float)(int8_t)(w2[h] >> 24);
              v[4 * c + 2 * h] = pack_bf16(f0, f1); v[4 * c + 2 * h + 1] = pack_bf16(f2, f3);
            }
          } else {
            const uint4 t = (j < D && kvalid) ? __ldg(src + (j >> 3)) : make_uint4(0, 0, 0, 0);
            v[4 * c] = t.x; v[4 * c + 1] = t.y; v[4 * c + 2] = t.z; v[4 * c + 3] = t.w;
          }
        }
        store_row_sw128(KVs + s * FP_SLAB, tid, v);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t da = make_sdesc_k_sw128(gm_smem_u32(Qs + (kk >> 2) * FP_SLAB)) + (uint64_t)(2 * (kk & 3));
        const uint64_t db = make_sdesc_k_sw128(gm_smem_u32(KVs + (kk >> 2) * FP_SLAB)) + (uint64_t)(2 * (kk & 3));
        umma_bf16(tmem, da, db, idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit(&bar_s);
    }
    ok = gm_wait(&bar_s, phase);
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- V tile -> V^T (the K buffer is free: S is complete) --------------------------------------
    {
      const uint4* src = (const uint4*)(p.v_cache + cbase);
      const int slab = tid >> 6, kc = tid & 63;           // key column inside the slab
      uint8_t* vb = KVs + slab * FP_SLAB + (kc & 7) * 2;
      const int chunk = kc >> 3;
      const float vsc = (p.kv_q8 && kvalid) ? *(const float*)(v8 + D) : 0.f;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint32_t w[4];
        if (p.kv_q8) {
          const uint2 cw = kvalid ? __ldg((const uint2*)(v8 + 8 * c)) : make_uint2(0, 0);
          const uint32_t w2[2] = {cw.x, cw.y};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            w[2 * h] = pack_bf16(vsc * (float)(int8_t)(w2[h] & 0xFF), vsc * (float)(int8_t)((w2[h] >> 8) & 0xFF));
            w[2 * h + 1] = pack_bf16(vsc * (float)(int8_t)((w2[h] >> 16) & 0xFF), vsc * (float)(int8_t)(w2[h] >> 24));
          }
        } else {
          const uint4 t = kvalid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
          w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = 8 * c + e;                        // row of V^T
          const uint16_t h = (uint16_t)(e & 1 ? w[e >> 1] >> 16 : w[e >> 1] & 0xFFFFu);
          *(uint16_t*)(vb + (j >> 3) * 1024 + (j & 7) * 128 + ((chunk ^ (j & 7)) << 4)) = h;
        }
      }
    }
    // ---- softmax over my row of S ------------------------------------------------------------------
    // keys of this tile that my query may see: [vis_lo, vis_hi)
    const int vis_hi = qvalid ? min(min(qpos + 1, ctx) - k0, 128) : 0;
    const int vis_lo = p.window > 0 ? max(0, qpos - p.window + 1 - k0) : 0;
    float tmax = -INFINITY;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + t_lane + (uint32_t)c0, r);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < vis_hi && c0 + j >= vis_lo) tmax = fmaxf(tmax, __uint_as_float(r[j]) * sc);
    }
    const float mnew = fmaxf(mrow, tmax);
    const float corr = mnew == -INFINITY ? 1.f : exp2f(mrow - mnew);     // mrow = -inf on the first visible tile -> 0
    float tsum = 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t r[32], pw[16];
      tmem_ld32(tmem + t_lane + (uint32_t)c0, r);
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = (c0 + j < vis_hi && c0 + j >= vis_lo) ? exp2f(__uint_as_float(r[j]) * sc - mnew) : 0.f;
        const float p1 = (c0 + j + 1 < vis_hi && c0 + j + 1 >= vis_lo) ? exp2f(__uint_as_float(r[j + 1]) * sc - mnew) : 0.f;
        // the sum uses the bf16-rounded probabilities that the tensor core will multiply
        const uint32_t pk = pack_bf16(p0, p1);
        tsum += __uint_as_float(pk << 16) + __uint_as_float(pk & 0xFFFF0000u);
        pw[j >> 1] = pk;
      }
      uint8_t* base = Ps + (c0 >> 6) * FP_SLAB + (tid >> 3) * 1024 + (tid & 7) * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int ch = ((c0 & 63) >> 3) + c;
        *(uint4*)(base + ((ch ^ (tid & 7)) << 4)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      }
    }
    lrow = lrow * corr + tsum;
    mrow = mnew;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {                    // 128 keys = 8 slices of 16
        const uint64_t da = make_sdesc_k_sw128(gm_smem_u32(Ps + (kk >> 2) * FP_SLAB)) + (uint64_t)(2 * (kk & 3));
        const uint64_t db = make_sdesc_k_sw128(gm_smem_u32(KVs + (kk >> 2) * FP_SLAB)) + (uint64_t)(2 * (kk & 3));
        umma_bf16(tmem + 128u, da, db, idesc_o, kk > 0 ? 1u : 0u);
      }
      umma_commit(&bar_o);
    }
    ok = gm_wait(&bar_o, phase);
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // ---- O = O * corr + O_tile ------------------------------------------------------------------------
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 16) {
      uint32_t r[16];
      tmem_ld16(tmem + t_lane + 128u + (uint32_t)c0, r);
#pragma unroll
      for (int j = 0; j < 16; ++j) o[c0 + j] = o[c0 + j] * corr + __uint_as_float(r[j]);
    }
  }
  if (!ok) atomicExch(&g_prefill_attn_error, 3101);
  if (ok && qvalid) {
    const float inv = lrow > 0.f ? 1.f / lrow : 0.f;
    if (p.out_bf16) {
      __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (int64_t)qrow * p.ld_out + head * D;
#pragma unroll
      for (int j = 0; j < D; j += 8) {
        __nv_bfloat162 w[4] = {__floats2bfloat162_rn(o[j] * inv, o[j + 1] * inv), __floats2bfloat162_rn(o[j + 2] * inv, o[j + 3] * inv),
                               __floats2bfloat162_rn(o[j + 4] * inv, o[j + 5] * inv), __floats2bfloat162_rn(o[j + 6] * inv, o[j + 7] * inv)};
        *(uint4*)(dst + j) = *(const uint4*)w;
      }
    } else {
      float* dst = p.out + (int64_t)qrow * p.ld_out + head * D;
#pragma unroll
      for (int j = 0; j < D; j += 4) *(float4*)(dst + j) = make_float4(o[j] * inv, o[j + 1] * inv, o[j + 2] * inv, o[j + 3] * inv);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

template <int D>
int launch_prefill(const AttnPrefillParams& p, cudaStream_t st) {
  constexpr int NSLAB = (D + 63) / 64;
  const size_t smem = (size_t)(NSLAB + 4) * FP_SLAB + 1024;
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(attn_prefill_tcgen05_kernel<D>, smem, 0); e != cudaSuccess) return (int)e;
  dim3 grid((p.n_tokens + 127) / 128, p.n_heads);
  return (int)launch(attn_prefill_tcgen05_kernel<D>, grid, dim3(FP_THREADS), smem, st, p);
}


// ---- second implementation: 16 query rows per CTA on mma.sync, K/V through a bulk-copy ring ----------------------------
// The tcgen05 kernel above walks the key tiles of a 128-query tile in one serial chain (load, MMA, transpose, softmax, MMA).
// This one cuts the chunk into tiles of 16 consecutive queries of one head: the four warps of a CTA take the 32-key stages of
// the tile's causal range in turn, each with its own ring slot filled by `cp.async.bulk` (same slot layout and fragment
// loads as the tensor-core decode kernel, attention_decode_body.cuh), and their partial results are merged through shared
// memory.  K/V of a layer's chunk stay in L2, so reading them once per 16 queries costs little, and the grid (chunk / 16 x
// heads CTAs of short independent chains) keeps every SM busy.  bf16 caches only.
constexpr int PM_WARPS = 4, PM_ROWS = 16;

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(const __grid_constant__ AttnPrefillParams p) {
  constexpr bool PAGE_COPY = HD == 80;
  constexpr int KS = HD / 16, NTL = HD / 8, RS = PAGE_COPY ? 2 * HD : 2 * HD + 16, SLOT = 64 * RS;
  extern __shared__ __align__(128) uint8_t pm_ring[];
  __shared__ float q_s[PM_ROWS][HD];
  __shared__ float part_s[PM_WARPS][PM_ROWS][HD + 2];
  __shared__ unsigned long long full[PM_WARPS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int m0 = blockIdx.x * PM_ROWS, head = blockIdx.y, kvh = head / (p.n_heads / p.n_kv_heads);
  pdl_launch_dependents();
  pdl_wait();
  const int pos0 = p.pos0_ptr ? *p.pos0_ptr : p.pos0;
  for (int i = tid; i < PM_ROWS * HD; i += 128) {
    const int r = i / HD, j = i - r * HD;
    q_s[r][j] = m0 + r < p.n_tokens ? p.qkv[(int64_t)(m0 + r) * p.ld_qkv + p.q_off + head * HD + j] : 0.f;
  }
  if (tid == 0) {
    for (int i = 0; i < PM_WARPS; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(att_smem_u32(&full[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int ctx = pos0 + p.n_tokens;
  const int qpos0 = pos0 + m0;                                     // position of row 0; row r sits at qpos0 + r
  const int end = min(ctx, qpos0 + PM_ROWS);                         // causal: no key beyond the tile's last query
  const int start = p.window > 0 ? max(0, qpos0 - p.window + 1) / ATT_PAGE * ATT_PAGE : 0;
  const int iters = (end - start + 31) / 32;
  uint8_t* slot = pm_ring + (size_t)warp * SLOT;
  unsigned long long* fb = &full[warp];
  auto issue = [&](int it) {
    const int tok0 = start + it * 32, nvalid = min(32, end - tok0);
    if (PAGE_COPY) {
      const int np = (nvalid + ATT_PAGE - 1) / ATT_PAGE;
      if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(fb)), "r"((uint32_t)(np * 2 * ATT_PAGE * RS)) : "memory");
      __syncwarp();
      if (lane < 4 && (lane & 1) < np) {
        const int tok = tok0 + (lane & 1) * ATT_PAGE;
        const int64_t boff = ((int64_t)p.page_table[tok / ATT_PAGE] * p.n_kv_heads + kvh) * ATT_PAGE * RS;
        const uint8_t* src = (lane & 2 ? (const uint8_t*)p.v_cache : (const uint8_t*)p.k_cache) + boff;
        att_bulk_g2s(slot + ((lane & 2 ? 32 : 0) + (lane & 1) * ATT_PAGE) * RS, src, ATT_PAGE * RS, fb);
      }
      return;
    }
    if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(fb)), "r"((uint32_t)(nvalid * 4 * HD)) : "memory");
    __syncwarp();
    if (lane < nvalid) {
      const int tok = tok0 + lane;
      const int64_t rowi = ((int64_t)p.page_table[tok / ATT_PAGE] * p.n_kv_heads + kvh) * ATT_PAGE + (tok % ATT_PAGE);
      att_bulk_g2s(slot + lane * RS, (const uint8_t*)p.k_cache + rowi * (2 * HD), 2 * HD, fb);
      att_bulk_g2s(slot + (32 + lane) * RS, (const uint8_t*)p.v_cache + rowi * (2 * HD), 2 * HD, fb);
    }
  };
  if (warp < iters) issue(warp);
  // Q fragments of rows gq and gq + 8 (bf16 head + remainder), pre-scaled for exp2
  const float qscale = p.scale * 1.4426950408889634f;
  uint32_t qa[KS][4], qb[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int f = 0; f < 4; ++f) {                                     // a0: (gq, lo cols), a1: (gq + 8, lo), a2: (gq, hi), a3: (gq + 8, hi)
      const int r = gq + 8 * (f & 1), jq = ks * 16 + 2 * tq + 8 * (f >> 1);
      const float f0 = q_s[r][jq] * qscale, f1 = q_s[r][jq + 1] * qscale;
      const uint32_t hi = att_pack_bf16(f0, f1);
      qa[ks][f] = hi;
      qb[ks][f] = att_pack_bf16(f0 - __uint_as_float(hi << 16), f1 - __uint_as_float(hi & 0xFFFF0000u));
    }
  }
  float o[NTL][4];
#pragma unroll
  for (int n = 0; n < NTL; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};
  int vend[2], vlo[2];                                                // keys visible to my two rows: [vlo, vend)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gq + 8 * h;
    vend[h] = m0 + r < p.n_tokens ? min(ctx, qpos0 + r + 1) : 0;
    vlo[h] = p.window > 0 ? max(0, qpos0 + r - p.window + 1) : 0;
  }
  bool ok = true;
  for (int it = warp; it < iters; it += PM_WARPS) {
    const int tok0 = start + it * 32;
    const uint32_t parity = (uint32_t)(it / PM_WARPS) & 1u;
    bool arrived = false;
    const uint32_t limit = ok ? ATT_WAIT_LIMIT : 1024u;
    for (uint32_t spin = 0; spin < limit; ++spin) if (att_try_wait(fb, parity)) { arrived = true; break; }
    if (!arrived) { ok = false; atomicExch(&g_prefill_attn_error, 3102); }
    if (tok0 + lane >= end || !ok) {                                  // rows past the end hold stale bytes
      uint4* kr4 = (uint4*)(slot + lane * RS); uint4* vr4 = (uint4*)(slot + (32 + lane) * RS);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) { kr4[c] = make_uint4(0, 0, 0, 0); vr4[c] = make_uint4(0, 0, 0, 0); }
    }
    __syncwarp();
    float sacc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const uint8_t* kp = slot + (8 * n + gq) * RS + (ks * 16 + 2 * tq) * 2;
        const uint32_t b0 = *(const uint32_t*)kp, b1 = *(const uint32_t*)(kp + 16);
        att_mma_bf16(sacc[n], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        att_mma_bf16(sacc[n], qb[ks][0], qb[ks][1], qb[ks][2], qb[ks][3], b0, b1);
      }
    }
    uint32_t pa[2][4];
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {                                     // row gq (c0, c1) and row gq + 8 (c2, c3)
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + 8 * n + 2 * tq + e;
          if (tok < vend[h] && tok >= vlo[h]) mx = fmaxf(mx, sacc[n][2 * h + e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const float mnew = fmaxf(mrow[h], mx);
      corr[h] = mnew == -INFINITY ? 1.f : exp2f(mrow[h] - mnew);
      float psum = 0.f;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int tok = tok0 + 8 * n + 2 * tq;
        const float p0 = (tok < vend[h] && tok >= vlo[h]) ? exp2f(sacc[n][2 * h] - mnew) : 0.f;
        const float p1 = (tok + 1 < vend[h] && tok + 1 >= vlo[h]) ? exp2f(sacc[n][2 * h + 1] - mnew) : 0.f;
        const uint32_t pk = att_pack_bf16(p0, p1);
        psum += __uint_as_float(pk << 16) + __uint_as_float(pk & 0xFFFF0000u);
        pa[n >> 1][(n & 1) * 2 + h] = pk;                             // k step n / 2: a0 / a1 from the even tile, a2 / a3 from the odd one
      }
      lsum[h] = lsum[h] * corr[h] + psum;
      mrow[h] = mnew;
    }
#pragma unroll
    for (int n = 0; n < NTL; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int n = 0; n < NTL; n += 2) {
        uint32_t r[4];
        const uint8_t* vrow = slot + (32 + 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7)) * RS + (n + (lane >> 4)) * 16;
        att_ldmatrix_x4_trans(r, vrow);
        att_mma_bf16(o[n], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], r[0], r[1]);
        att_mma_bf16(o[n + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], r[2], r[3]);
      }
    }
    __syncwarp();
    if (it + PM_WARPS < iters) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(it + PM_WARPS);
    }
  }
  // ---- the four warps' partial results of every row meet in shared memory ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = lsum[h];
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);
    const int r = gq + 8 * h;
#pragma unroll
    for (int n = 0; n < NTL; ++n) { part_s[warp][r][8 * n + 2 * tq] = o[n][2 * h]; part_s[warp][r][8 * n + 2 * tq + 1] = o[n][2 * h + 1]; }
    if (tq == 0) { part_s[warp][r][HD] = mrow[h]; part_s[warp][r][HD + 1] = l; }
  }
  __syncthreads();
  for (int i = tid; i < PM_ROWS * HD; i += 128) {
    const int r = i / HD, j = i - r * HD;
    if (m0 + r >= p.n_tokens) continue;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < PM_WARPS; ++w) mm = fmaxf(mm, part_s[w][r][HD]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < PM_WARPS; ++w) {
      const float mw = part_s[w][r][HD];
      const float c = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      a += c * part_s[w][r][j]; ll += c * part_s[w][r][HD + 1];
    }
    const float v = ll > 0.f ? a / ll : 0.f;
    const int64_t off = (int64_t)(m0 + r) * p.ld_out + head * HD + j;
    if (p.out_bf16) ((__nv_bfloat16*)p.out)[off] = __float2bfloat16_rn(v); else p.out[off] = v;
  }
}

template <int HD>
int launch_prefill_mma(const AttnPrefillParams& p, cudaStream_t st) {
  const size_t ring = (size_t)PM_WARPS * 64 * (HD == 80 ? 2 * HD : 2 * HD + 16);
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(attn_prefill_mma_kernel<HD>, ring, 0); e != cudaSuccess) return (int)e;
  dim3 grid((p.n_tokens + PM_ROWS - 1) / PM_ROWS, p.n_heads);
  return (int)launch(attn_prefill_mma_kernel<HD>, grid, dim3(128), ring, st, p);
}

}  // namespace rlz

extern "C" {

int rlz_attn_prefill_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, rlz::g_prefill_attn_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) { int z = 0; cudaMemcpyToSymbol(rlz::g_prefill_attn_error, &z, sizeof(int)); }
  return v;
}

// 1 when the tensor-core prefill kernel has an instantiation for this head size
int rlz_attn_prefill_supported(int head_dim) { return head_dim == 64 || head_dim == 80 || head_dim == 96 || head_dim == 128; }

// impl: -1 = the default choice (or RLZ_PREFILL_ATT), 0 = tcgen05 kernel, 1 = mma.sync kernel (bf16 caches only)
int rlz_attn_prefill_impl(const rlz::AttnPrefillParams* pp, void* stream, int impl) {
  using namespace rlz;
  const AttnPrefillParams& p = *pp;
  if (p.n_tokens < 1 || p.n_kv_heads < 1 || p.n_heads % p.n_kv_heads || p.pos0 < 0 || p.window < 0) return -2;
  if (((uintptr_t)p.k_cache & 15) || ((uintptr_t)p.v_cache & 15) || ((uintptr_t)p.out & 15) || (p.ld_out & (p.out_bf16 ? 7 : 3)) || (p.head_dim & 7)) return -4;
  cudaStream_t st = (cudaStream_t)stream;
  // implementation: "mma" (16-query tiles on mma.sync, bf16 caches) or "tc" (128-query tiles on tcgen05, also int8 caches);
  // RLZ_PREFILL_ATT forces one
  static const int impl_env = [] { const char* e = getenv("RLZ_PREFILL_ATT"); return !e ? -1 : (e[0] == 'm' ? 1 : 0); }();
  // default: mma where whole pages can be copied (head_dim 80: TTFT of a 512-token Phi-2-shaped prompt 8.0 vs 9.1 ms); with
  // row-by-row copies (head_dim 128, 1024-token Llama-3-8B-shaped prompt) the two measured the same (35.9 vs 35.2 ms)
  const int want = impl >= 0 ? impl : impl_env;
  if (want == 1 && p.kv_q8) return -5;
  const bool use_mma = !p.kv_q8 && (want < 0 ? p.head_dim == 80 : want == 1);
  if (use_mma) {
    switch (p.head_dim) {
      case 64: return launch_prefill_mma<64>(p, st);
      case 80: return launch_prefill_mma<80>(p, st);
      case 96: return launch_prefill_mma<96>(p, st);
      case 128: return launch_prefill_mma<128>(p, st);
      default: return -1;
    }
  }
  switch (p.head_dim) {
    case 64: return launch_prefill<64>(p, st);
    case 80: return launch_prefill<80>(p, st);
    case 96: return launch_prefill<96>(p, st);
    case 128: return launch_prefill<128>(p, st);
    default: return -1;
  }
}

int rlz_attn_prefill(const rlz::AttnPrefillParams* pp, void* stream) { return rlz_attn_prefill_impl(pp, stream, -1); }

int rlz_sizeof_attn_prefill_params() { return (int)sizeof(rlz::AttnPrefillParams); }

}  // extern "C"
