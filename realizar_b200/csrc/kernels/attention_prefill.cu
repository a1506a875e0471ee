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

  // ---- Q tile: my row, fp32 -> bf16, swizzled --------------------------------------------------
  const int qrow = m0 + tid;
  const bool qvalid = qrow < p.n_tokens;
  const int qpos = p.pos0 + qrow;
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
  const int ctx = p.pos0 + p.n_tokens;
  const int kend = min(ctx, p.pos0 + m0 + 128);          // causal: no key beyond the tile's last query
  const int klo = p.window > 0 ? max(0, p.pos0 + m0 - p.window + 1) / 128 * 128 : 0;
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
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((p.n_tokens + 127) / 128, p.n_heads);
  return (int)launch(attn_prefill_tcgen05_kernel<D>, grid, dim3(FP_THREADS), smem, st, p);
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

int rlz_attn_prefill(const rlz::AttnPrefillParams* pp, void* stream) {
  using namespace rlz;
  const AttnPrefillParams& p = *pp;
  if (p.n_tokens < 1 || p.n_kv_heads < 1 || p.n_heads % p.n_kv_heads || p.pos0 < 0 || p.window < 0) return -2;
  if (((uintptr_t)p.k_cache & 15) || ((uintptr_t)p.v_cache & 15) || ((uintptr_t)p.out & 15) || (p.ld_out & (p.out_bf16 ? 7 : 3)) || (p.head_dim & 7)) return -4;
  cudaStream_t st = (cudaStream_t)stream;
  switch (p.head_dim) {
    case 64: return launch_prefill<64>(p, st);
    case 80: return launch_prefill<80>(p, st);
    case 96: return launch_prefill<96>(p, st);
    case 128: return launch_prefill<128>(p, st);
    default: return -1;
  }
}

int rlz_sizeof_attn_prefill_params() { return (int)sizeof(rlz::AttnPrefillParams); }

}  // extern "C"
