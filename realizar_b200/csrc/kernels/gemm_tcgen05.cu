// Dequant-GEMM on the 5th-generation tensor cores: Y[M, N] (+)= X[M, K] . W[N, K]^T with W in a
// K-quant block layout (Q4_K / Q5_K / Q6_K) or dense bf16/f16, X in bf16, fp32 accumulation in
// tensor memory.  Used for prefill and for decode batches too large for the GEMV kernels.
//
// One CTA (128 threads) owns 128 weight rows x MT tokens (x one K split):
//   * every thread dequantises 64 weights of "its" row per K step straight into shared memory as
//     bf16 in the K-major 128-byte-swizzled layout that tcgen05.mma reads (operand A), and copies
//     64 activations of "its" token the same way (operand B);
//   * one elected thread issues four tcgen05.mma (M=128, N=MT, K=16) per K step and commits them
//     to an mbarrier; the two shared-memory stages alternate, so dequantisation of step s+1
//     overlaps the tensor-core work of step s;
//   * the accumulator lives in TMEM (MT columns); the epilogue reads it back with tcgen05.ld,
//     applies bias / activation / residual and stores (or atomically adds, with split-K) fp32.
// Every mbarrier wait is bounded; on expiry the CTA records error 3001, releases its tensor
// memory and returns.
//
// Replaces the reference's q4k/q5k/q6k_gemm_ggml, tensor_core_q4k_gemm (WMMA), dp4a_q4k_gemm,
// dequant-to-f16/f32 + cuBLAS HGEMM/SGEMM and cuBLASLt FP8 call sites
// (src/cuda/executor/layers/cublas_prefill/gemm.rs:70-1100).
#include "common.cuh"
#include "../gemv_blocks.h"
#include <cuda_bf16.h>

namespace rlz {

__device__ int g_gemm_error = 0;

constexpr int GM_THREADS = 128;
constexpr int GM_ROWS = 128;          // weight rows per CTA = MMA M
constexpr int GM_KSTEP = 64;          // K elements per stage (one 128-byte swizzle row of bf16)
constexpr uint32_t GM_WAIT_LIMIT = 1u << 24;

struct GemmParams {
  const uint8_t* W; int64_t w_stride; int32_t qtype; int32_t n; int32_t k; int32_t m;
  const __nv_bfloat16* X; int64_t ldx;
  float* Y; int64_t ldy;
  const float* bias; const float* residual; int64_t ld_res;
  int32_t act; int32_t splitk; int32_t atomic_out; int32_t _pad;
};

__device__ __forceinline__ uint32_t gm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_sdesc_k_sw128(uint32_t smem_addr) {
  // K-major, SWIZZLE_128B: rows of 128 bytes, 8-row groups 1024 bytes apart
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);            // start address
  d |= (uint64_t)1 << 16;                                  // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                                  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                                  // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t make_idesc_bf16(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(gm_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool gm_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(gm_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool gm_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < GM_WAIT_LIMIT; ++i) if (gm_try_wait(bar, parity)) return true;
  return false;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *(const uint32_t*)&v;
}

// 64 weights of one row starting at column k0 (multiple of 64) as 32 packed bf16 pairs
__device__ __forceinline__ void dequant_row64(const uint8_t* row, int qtype, int k0, uint32_t* out) {
  const int sb = k0 >> 8, g = (k0 >> 6) & 3;
  if (qtype == QT_Q4_K || qtype == QT_Q5_K) {
    const int bb = qtype == QT_Q4_K ? 144 : 176;
    const uint8_t* blk = row + (int64_t)sb * bb;
    const uint4 hdr = __ldg((const uint4*)blk);
    const float d = h2f_alu(hdr.x & 0xFFFFu), dmin = h2f_alu(hdr.x >> 16);
    const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
    const float d0 = d * (float)k4_pick(ks.sc_lo, ks.sc_hi, 2 * g), d1 = d * (float)k4_pick(ks.sc_lo, ks.sc_hi, 2 * g + 1);
    const float m0 = dmin * (float)k4_pick(ks.m_lo, ks.m_hi, 2 * g), m1 = dmin * (float)k4_pick(ks.m_lo, ks.m_hi, 2 * g + 1);
    const uint8_t* qs = blk + (qtype == QT_Q4_K ? 16 : 48) + 32 * g;
    const uint4 q0 = __ldg((const uint4*)qs), q1 = __ldg((const uint4*)(qs + 16));
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint32_t hw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (qtype == QT_Q5_K) {
      const uint4 h0 = __ldg((const uint4*)(blk + 16)), h1 = __ldg((const uint4*)(blk + 32));
      hw[0] = h0.x; hw[1] = h0.y; hw[2] = h0.z; hw[3] = h0.w; hw[4] = h1.x; hw[5] = h1.y; hw[6] = h1.z; hw[7] = h1.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {                         // word i holds elements 4i..4i+3 (low nibbles) and 32+4i.. (high)
      float lo[4], hi[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        int ql = (qw[i] >> (8 * b)) & 0xF, qh = (qw[i] >> (8 * b + 4)) & 0xF;
        if (qtype == QT_Q5_K) { ql |= ((hw[i] >> (8 * b + 2 * g)) & 1) << 4; qh |= ((hw[i] >> (8 * b + 2 * g + 1)) & 1) << 4; }
        lo[b] = d0 * (float)ql - m0; hi[b] = d1 * (float)qh - m1;
      }
      out[2 * i] = pack_bf16(lo[0], lo[1]); out[2 * i + 1] = pack_bf16(lo[2], lo[3]);
      out[16 + 2 * i] = pack_bf16(hi[0], hi[1]); out[16 + 2 * i + 1] = pack_bf16(hi[2], hi[3]);
    }
  } else if (qtype == QT_Q6_K) {
    // the 64 columns [64g', 64g'+64) of a block: half n = g >> 1, positions 64*(g&1) .. +63 within the half
    const uint8_t* blk = row + (int64_t)sb * Q6K_DEV_STRIDE;
    const int n = g >> 1, upper = g & 1;                  // upper: elements 64..127 of the half use the high nibbles
    const float d = h2f_alu((uint32_t)blk[208] | ((uint32_t)blk[209] << 8));
    const int8_t* sc = (const int8_t*)(blk + 192 + 8 * n + 4 * upper);     // scales of the four 16-chunks
#pragma unroll
    for (int part = 0; part < 2; ++part) {                // 32 elements each: l = 0..31 of ql[l] / ql[l+32]
      const uint8_t* ql = blk + 64 * n + 32 * part;
      const uint8_t* qh = blk + 128 + 32 * n;
      const float s0 = d * (float)sc[2 * part], s1 = d * (float)sc[2 * part + 1];
#pragma unroll
      for (int w4 = 0; w4 < 8; ++w4) {
        const uint32_t lw = __ldg((const uint32_t*)(ql + 4 * w4)), hwv = __ldg((const uint32_t*)(qh + 4 * w4));
        float v[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int l = 4 * w4 + b;
          const int nib = upper ? ((lw >> (8 * b + 4)) & 0xF) : ((lw >> (8 * b)) & 0xF);
          const int hb = (hwv >> (8 * b + 2 * (2 * upper + part))) & 3;
          v[b] = (l < 16 ? s0 : s1) * (float)((nib | (hb << 4)) - 32);
        }
        out[16 * part + 2 * w4] = pack_bf16(v[0], v[1]); out[16 * part + 2 * w4 + 1] = pack_bf16(v[2], v[3]);
      }
    }
  } else if (qtype == QT_BF16) {
    const uint4* src = (const uint4*)(row + (int64_t)k0 * 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) { const uint4 t = __ldg(src + i); out[4 * i] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w; }
  } else {                                                // F16
    const uint4* src = (const uint4*)(row + (int64_t)k0 * 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 t = __ldg(src + i); const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) out[4 * i + j] = pack_bf16(h2f_alu(w[j] & 0xFFFFu), h2f_alu(w[j] >> 16));
    }
  }
}

// store 64 bf16 (32 words) as row r of a [rows x 64] K-major SWIZZLE_128B tile
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int r, const uint32_t* v) {
  uint8_t* base = tile + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *(uint4*)(base + ((c ^ (r & 7)) << 4)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

template <int MT>
__global__ void __launch_bounds__(GM_THREADS) gemm_kquant_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t gsm[];
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * GM_ROWS, m0 = blockIdx.y * MT;
  // shared memory: 2 stages x (A tile 128 x 64 bf16 = 16 KB, B tile MT x 64 bf16)
  uint8_t* sm = (uint8_t*)(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = GM_ROWS * 128, B_BYTES = MT * 128, STAGE = A_BYTES + B_BYTES;

  if (tid == 0) {
    failed_s = 0;
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gm_smem_u32(&bar[1])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {                                        // one warp allocates MT columns of tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem_u32(&tmem_base_s)), "r"((uint32_t)(MT < 32 ? 32 : MT)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();

  // K range of this split
  const int ksteps_total = p.k / GM_KSTEP;
  const int per = (ksteps_total + p.splitk - 1) / p.splitk;
  const int ks0 = blockIdx.z * per, ks1 = min(ksteps_total, ks0 + per);
  const uint32_t idesc = make_idesc_bf16(GM_ROWS, MT);
  const int wrow = n0 + tid;                              // my weight row
  const uint8_t* wptr = p.W + (int64_t)min(wrow, p.n - 1) * p.w_stride;
  bool ok = true;

  for (int ks = ks0, it = 0; ks < ks1; ++ks, ++it) {
    const int s = it & 1;
    if (it >= 2) {                                        // stage s is free once the MMAs issued two steps ago completed
      ok = ok && gm_wait(&bar[s], (uint32_t)((it >> 1) - 1) & 1u);
      if (!ok) break;
    }
    uint8_t* At = sm + s * STAGE;
    uint8_t* Bt = At + A_BYTES;
    uint32_t v[32];
    if (wrow < p.n) dequant_row64(wptr, p.qtype, ks * GM_KSTEP, v);
    else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0u;
    }
    store_row_sw128(At, tid, v);
    for (int t = tid; t < MT; t += GM_THREADS) {          // activations: token t of this tile
      const int tok = m0 + t;
      if (tok < p.m) {
        const uint4* src = (const uint4*)(p.X + (int64_t)tok * p.ldx + (int64_t)ks * GM_KSTEP);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const uint4 x4 = src[i]; v[4 * i] = x4.x; v[4 * i + 1] = x4.y; v[4 * i + 2] = x4.z; v[4 * i + 3] = x4.w; }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      store_row_sw128(Bt, t, v);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy writes -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t da = make_sdesc_k_sw128(gm_smem_u32(At)), db = make_sdesc_k_sw128(gm_smem_u32(Bt));
#pragma unroll
      for (int kk = 0; kk < GM_KSTEP / 16; ++kk)          // advance 32 bytes (two 16-byte units) per K=16 slice
        umma_bf16(tmem_d, da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), idesc, (it > 0 || kk > 0) ? 1u : 0u);
      umma_commit(&bar[s]);
    }
  }
  // wait for the last commits of both stages
  const int nit = max(0, ks1 - ks0);
  if (ok && nit >= 1) { const int it = nit - 1; ok = gm_wait(&bar[it & 1], (uint32_t)(it >> 1) & 1u); }
  if (ok && nit >= 2) { const int it = nit - 2; ok = gm_wait(&bar[it & 1], (uint32_t)(it >> 1) & 1u); }
  if (!ok) { failed_s = 1; atomicExch(&g_gemm_error, 3001); }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- epilogue: TMEM lane = weight row, column = token --------------------------------------
  if (ok && nit > 0) {
    const int row = n0 + warp * 32 + lane;
    const float bias = (p.bias && row < p.n && blockIdx.z == 0) ? p.bias[row] : 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < MT; c0 += 32) {
      uint32_t r[32];
      const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
            "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
            "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
          : "r"(taddr) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < p.n) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = m0 + c0 + j;
          if (tok < p.m) {
            float v = __uint_as_float(r[j]) + bias;
            float* dst = p.Y + (int64_t)tok * p.ldy + row;
            if (p.atomic_out) atomicAdd(dst, v);
            else {
              if (p.act == ACT_GELU) v = gelu_tanh(v); else if (p.act == ACT_SILU) v = silu(v);
              if (p.residual) v += p.residual[(int64_t)tok * p.ld_res + row];
              *dst = v;
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)(MT < 32 ? 32 : MT)) : "memory");
}

template <int MT>
cudaError_t launch_gemm(const GemmParams& p, cudaStream_t st) {
  const size_t smem = 2 * (GM_ROWS * 128 + MT * 128) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kquant_tcgen05_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((p.n + GM_ROWS - 1) / GM_ROWS, (p.m + MT - 1) / MT, p.splitk);
  return launch(gemm_kquant_tcgen05_kernel<MT>, grid, dim3(GM_THREADS), smem, st, p);
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

// Y[m, n] = act(X[m, k] W^T + bias) + residual.  With splitk > 1 the partial products are added
// atomically into Y, which the caller must have initialised (zeros, or the residual); bias is added
// by split 0 and no activation is applied.  Returns 0, a negative code for bad arguments or a cudaError_t.
int rlz_gemm_kquant(const rlz::GemmParams* pp, void* stream) {
  using namespace rlz;
  GemmParams p = *pp;
  if (p.k % GM_KSTEP || p.m < 1 || p.n < 1) return -1;
  if (!(p.qtype == QT_Q4_K || p.qtype == QT_Q5_K || p.qtype == QT_Q6_K || p.qtype == QT_BF16 || p.qtype == QT_F16)) return -2;
  if ((p.qtype == QT_Q4_K || p.qtype == QT_Q5_K || p.qtype == QT_Q6_K) && p.k % 256) return -3;
  if (((uintptr_t)p.X & 15) || (p.ldx % 8) || ((uintptr_t)p.W & 15) || (p.w_stride & 15)) return -4;
  if (p.splitk < 1) p.splitk = 1;
  if (p.splitk > p.k / GM_KSTEP) p.splitk = p.k / GM_KSTEP;
  p.atomic_out = p.splitk > 1 ? 1 : 0;
  if (p.atomic_out && p.act != ACT_NONE) return -5;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (p.m <= 32) e = launch_gemm<32>(p, st);
  else if (p.m <= 64) e = launch_gemm<64>(p, st);
  else e = launch_gemm<128>(p, st);
  return (int)e;
}

}  // extern "C"
