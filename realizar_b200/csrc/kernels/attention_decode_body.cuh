// Flash-decode attention job as a device function (see attention_decode.cu for the description of the algorithm).
// Used by the standalone kernel and by the persistent decode-step kernel.
#pragma once
#include "common.cuh"
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <math.h>

namespace rlz {

namespace cg = cooperative_groups;

constexpr int ATT_PAGE = 16;
constexpr int ATT_THREADS = 128;     // 8 half-warps; each takes up to TB tokens per iteration (TB by head-group size, below)
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_PT_MAX = 64;       // page-table entries of a split staged in shared memory (1024 tokens)
constexpr int ATT_MAX_CLUSTER = 8;   // portable cluster size
constexpr int ATT_RING = 4;          // streamed mode: ring stages of two pages (32 tokens) of K and V each
constexpr uint32_t ATT_WAIT_LIMIT = 1u << 22;
enum { MERGE_GLOBAL = 0, MERGE_CLUSTER = 1, MERGE_NONE = 2 };

struct AttnDecodeParams {
  const float* qkv;        // [B, ld_qkv]: q heads | k heads | v heads (after bias)
  float* out;              // [B, ld_out]: attention output, head-major
  __nv_bfloat16* k_cache;     // bf16 rows, or int8 rows when kv_q8 (see below)
  __nv_bfloat16* v_cache;
  const int32_t* positions;   // [B]
  const int32_t* page_table;  // [B, max_pages]
  const float* q_norm_w;   // [head_dim] or null
  const float* k_norm_w;   // [head_dim] or null
  float* partial;          // scratch [B, H, splits, head_dim + 2]
  int32_t* counters;       // scratch [B, n_kv_heads * head_groups], zero before first use
  int64_t ld_qkv, ld_out;
  int32_t n_heads, n_kv_heads, head_dim, max_pages;
  int32_t rope_dim, rope_type, splits, batch;
  int32_t q_off, k_off, v_off;         // element offsets of the q / k / v sections in a qkv row
  int32_t pt_stride;                   // page_table elements between batch rows (0: every row shares one table)
  float rope_theta, eps, scale;
  int32_t no_append;                   // 1: the new rows are already in the cache (prefill), only attend
  int32_t window;                      // > 0: attend to positions (pos - window, pos] only
  int32_t rope_table_len;              // positions covered by rope_table
  const float2* rope_table;            // [rope_table_len, rope_dim / 2] (cos, sin) or null
  int32_t kv_q8;                       // 1: int8 cache rows of head_dim + 16 bytes (codes, then the fp32 scale of the row)
  int32_t num_pages;                   // pages in the cache (0: unknown, page ids are not checked)
};

// ---- int8 KV rows: [head_dim codes][fp32 scale][12 bytes padding]; value = code * scale, scale = max|x| / 127 per (token, kv head) ----
__device__ __forceinline__ int kv_row_bytes(int d, int q8) { return q8 ? d + 16 : 2 * d; }
// four codes of a word -> floats: the biased byte goes into the mantissa of 2^23, the bias comes off exactly, then the scale
__device__ __forceinline__ void q8_word_to_float(uint32_t w, float sc, float* out) {
  const uint32_t b = w ^ 0x80808080u;                     // bias the code to 0..255; (2^23 + byte) - (2^23 + 128) is exact
  out[0] = (__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7540)) - 8388736.f) * sc;
  out[1] = (__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7541)) - 8388736.f) * sc;
  out[2] = (__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7542)) - 8388736.f) * sc;
  out[3] = (__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7543)) - 8388736.f) * sc;
}
__device__ __forceinline__ float q8_round(float x, float sc) {      // what the cache will return for x
  return sc > 0.f ? fminf(127.f, fmaxf(-127.f, rintf(x / sc))) * sc : 0.f;
}

__device__ __forceinline__ void rope_inplace(float* v, int d_rot, int rope_type, int pos, float theta, const float2* table, int tid, int nthreads) {
  const int half = d_rot >> 1;
  for (int i = tid; i < half; i += nthreads) {
    float sn, cs;
    if (table) {
      const float2 t = __ldg(table + (int64_t)pos * half + i);
      cs = t.x; sn = t.y;
    } else {
      const float freq = powf(theta, -2.f * (float)i / (float)d_rot);
      sincosf((float)pos * freq, &sn, &cs);
    }
    const int i0 = rope_type == 2 ? i : 2 * i, i1 = rope_type == 2 ? i + half : 2 * i + 1;
    const float a = v[i0], b = v[i1];
    v[i0] = a * cs - b * sn;
    v[i1] = a * sn + b * cs;
  }
}

// 3201: a streamed K/V stage never arrived (bounded wait ran out); 3301: a position beyond the page-table row (the sequence
// is skipped); 3302: a page id outside the cache (read as page 0, the append is skipped)
static __device__ int g_attn_decode_error = 0;
// page id from the table, checked against the cache size when the launcher knows it
__device__ __forceinline__ int att_page(const AttnDecodeParams& p, int raw) {
  if (p.num_pages > 0 && (unsigned)raw >= (unsigned)p.num_pages) { atomicExch(&g_attn_decode_error, 3302); return 0; }
  return raw;
}

__device__ __forceinline__ uint32_t att_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool att_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(att_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void att_bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(att_smem_u32(dst)), "l"(src), "r"(bytes), "r"(att_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t att_pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *(const uint32_t*)&v;
}
__device__ __forceinline__ void att_mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void att_ldmatrix_x4_trans(uint32_t* r, const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(att_smem_u32(row)) : "memory");
}

// Shared memory of one 128-thread attention job.
// MERGE_CLUSTER: up to 4 heads per CTA the splits PUSH their results into the gather buffer of cluster rank 0 and leave;
// with 8 heads the buffer would not fit in static shared memory and rank 0 pulls the peers' res_s instead
template <int GT, int MERGE> struct AttnSmem {
  static constexpr bool PUSH = MERGE == MERGE_CLUSTER && GT <= 4;
  float q_s[GT][128];
  float k_s[128], v_s[128];
  float part_s[ATT_WARPS][GT][128 + 2];   // per-warp partials
  float res_s[PUSH ? 1 : GT][128 + 2];
  float gat_s[PUSH ? ATT_MAX_CLUSTER : 1][PUSH ? GT : 1][128 + 2];
  int32_t pt_s[ATT_PT_MAX];               // physical pages of this split's token range
  float qs_s[2][ATT_THREADS / 32 + 1];    // int8 cache: max|k|, max|v| of the new row (per warp, then total)
  int last_flag;
  unsigned long long full[ATT_RING];      // streamed mode: one mbarrier per ring stage
};

// The work of one attention CTA: job (bx = kv head x head group, split, b = sequence), thread tid of 128.
// SUB = false: the 128 threads are a whole CTA (standalone kernel).  SUB = true: they are one quarter of a larger CTA of a
// persistent kernel and synchronise on the named barrier `bar`; only the global-memory merge modes are available there.
// TBO > 0 overrides the tokens taken per half-warp per iteration (register budget of the host kernel).
// DEEP = 2 ("streamed", for launches that fill the GPU many times over): the pages of the split are brought into a ring in
// shared memory (`ring`, ATT_RING stages of two pages of K and two of V) by bulk async copies, several stages ahead of the
// arithmetic, instead of being loaded into registers by the threads that use them.
// DEEP = 3 ("tensor-core", head_dim HD known at compile time, bf16 cache): every warp owns one ring slot of 32 token rows
// (padded to HD * 2 + 16 bytes so that fragment loads are conflict-free) and computes S = Q K^T and O += P V of its stages
// with mma.sync m16n8k16 (rows = the query heads of the group, padded to 16), about a seventh of the instructions per token
// of the scalar path; the warps' partial results meet in the same merge as the other modes.
// Tensor-core mode: request the 32 token rows of iteration `it` into warp `warp`'s ring slot - whole pages with one bulk copy each
// at head_dim 80, else one copy per K and V row (every lane its token's rows).
template <int HD>
__device__ __forceinline__ void att_mma_issue(const AttnDecodeParams& p, uint8_t* ring, unsigned long long* fb, int warp, int lane, int it, int start,
                                              int end, bool pt_staged, const int* pt_s, const int32_t* pt, int kvh) {
  constexpr bool PAGE_COPY = HD == 80;
  constexpr int RS = PAGE_COPY ? 2 * HD : 2 * HD + 16, SLOT = 64 * RS;
  uint8_t* slot = ring + (size_t)warp * SLOT;
  const int tok0 = start + it * 32, nvalid = min(32, end - tok0);
  if (PAGE_COPY) {
    const int np = (nvalid + ATT_PAGE - 1) / ATT_PAGE;                 // whole pages: lanes 0..3 = (K, V) x (page 0, page 1)
    if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(fb)), "r"((uint32_t)(np * 2 * ATT_PAGE * RS)) : "memory");
    __syncwarp();
    if (lane < 4 && (lane & 1) < np) {
      const int tok = tok0 + (lane & 1) * ATT_PAGE;
      const int page = pt_staged ? pt_s[(tok - start) / ATT_PAGE] : att_page(p, pt[tok / ATT_PAGE]);
      const int64_t boff = ((int64_t)page * p.n_kv_heads + kvh) * ATT_PAGE * RS;
      const uint8_t* src = (lane & 2 ? (const uint8_t*)p.v_cache : (const uint8_t*)p.k_cache) + boff;
      att_bulk_g2s(slot + ((lane & 2 ? 32 : 0) + (lane & 1) * ATT_PAGE) * RS, src, ATT_PAGE * RS, fb);
    }
    return;
  }
  if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(fb)), "r"((uint32_t)(nvalid * 4 * HD)) : "memory");
  __syncwarp();
  if (lane < nvalid) {
    const int tok = tok0 + lane;
    const int page = pt_staged ? pt_s[(tok - start) / ATT_PAGE] : att_page(p, pt[tok / ATT_PAGE]);
    const int64_t rowi = ((int64_t)page * p.n_kv_heads + kvh) * ATT_PAGE + (tok % ATT_PAGE);
    att_bulk_g2s(slot + lane * RS, (const uint8_t*)p.k_cache + rowi * (2 * HD), 2 * HD, fb);
    att_bulk_g2s(slot + (32 + lane) * RS, (const uint8_t*)p.v_cache + rowi * (2 * HD), 2 * HD, fb);
  }
}

// WAITS: the body itself waits for the preceding kernel (programmatic dependent launch), after the work that does not depend on
// it: in the tensor-core mode of a decode step the first K/V stage of every warp is requested before that wait - the cached
// rows were written by earlier steps, only the new row comes from the preceding GEMV and it is patched in from shared memory.
template <int GT, int MERGE, int DEEP, int Q8, int TBO, bool SUB, int HD = 0, bool WAITS = false>
__device__ __forceinline__ void attn_decode_body(const AttnDecodeParams& p, const int bx, const int split, const int b, const int tid,
                                                 AttnSmem<GT, MERGE>& sm, const int bar, uint8_t* ring = nullptr) {
#define ATT_SYNC() do { if (SUB) asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(ATT_THREADS) : "memory"); else __syncthreads(); } while (0)
  static_assert(!SUB || MERGE != MERGE_CLUSTER, "cluster merge needs one job per CTA");
  const int G = p.n_heads / p.n_kv_heads;
  const int hgroups = (G + GT - 1) / GT;
  const int kvh = bx / hgroups, hg = bx - kvh * hgroups;
  const int d = p.head_dim;
  const int g0 = hg * GT, gn = min(GT, G - g0);          // query heads [g0, g0+gn) of this kv head
  const int lane = tid & 31, warp = tid >> 5;
  const int l16 = lane & 15, hw = tid >> 4;              // half-warp id 0..7
  constexpr bool PUSH = AttnSmem<GT, MERGE>::PUSH;
  auto& q_s = sm.q_s; auto& k_s = sm.k_s; auto& v_s = sm.v_s; auto& part_s = sm.part_s; auto& res_s = sm.res_s; auto& gat_s = sm.gat_s;
  auto& pt_s = sm.pt_s; auto& qs_s = sm.qs_s; int& last_flag = sm.last_flag;

  const int pos = p.positions[b];
  if (pos < 0) { if constexpr (WAITS) pdl_wait(); return; }   // uniform over the cluster (same sequence); the grid still orders after its predecessor
  if (p.max_pages > 0 && pos / ATT_PAGE >= p.max_pages) {  // the position has run past the sequence's page-table row: touch nothing
    if (tid == 0) atomicExch(&g_attn_decode_error, 3301);
    if constexpr (WAITS) pdl_wait();
    return;
  }
  if (PUSH) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");     // phase 1: "I have started"; waited on before the push
  const int seq_len = pos + 1;
  const int lo = p.window > 0 ? max(0, seq_len - p.window) : 0;      // first position attended to
  const int lo_al = lo / ATT_PAGE * ATT_PAGE;
  int chunk = (seq_len - lo_al + p.splits - 1) / p.splits;
  chunk = (chunk + ATT_PAGE - 1) / ATT_PAGE * ATT_PAGE;
  const int start = lo_al + split * chunk, end = min(seq_len, start + chunk);
  const bool owner = !p.no_append && start <= pos && pos < end;

  // ---- stage the split's page-table entries, q (this head group), and k/v of the new token: independent loads ----
  const int32_t* pt = p.page_table + (int64_t)b * p.pt_stride;
  const int npages = (max(0, end - start) + ATT_PAGE - 1) / ATT_PAGE;
  const bool pt_staged = npages <= ATT_PT_MAX;
  if (pt_staged && tid < npages) pt_s[tid] = att_page(p, pt[start / ATT_PAGE + tid]);
  bool prefetched = false;
  if constexpr (DEEP == 3 && WAITS) {
    // rows appended by a kernel that runs right before this one (token-batch passes: no_append) must be waited for first
    prefetched = !p.no_append;
    if (tid == 0) {
      for (int i = 0; i < ATT_RING; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(att_smem_u32(&sm.full[i])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    ATT_SYNC();                                            // barriers initialised, page-table entries staged
    if (prefetched && warp < (max(0, end - start) + 31) / 32)
      att_mma_issue<HD>(p, ring, &sm.full[warp], warp, lane, warp, start, end, pt_staged, pt_s, pt, kvh);
    pdl_wait();
  }
  const float* row = p.qkv + (int64_t)b * p.ld_qkv;
  for (int i = tid; i < gn * d; i += ATT_THREADS) {
    const int g = i / d, j = i - g * d;
    q_s[g][j] = row[p.q_off + (kvh * G + g0 + g) * d + j];
  }
  if (owner) {
    for (int j = tid; j < d; j += ATT_THREADS) {
      k_s[j] = row[p.k_off + kvh * d + j];
      v_s[j] = row[p.v_off + kvh * d + j];
    }
  }
  ATT_SYNC();
  if (p.q_norm_w) {      // per-head RMSNorm, one warp per head
    for (int g = warp; g < gn + (owner ? 1 : 0); g += ATT_THREADS / 32) {
      float* v = g < gn ? q_s[g] : k_s;
      const float* w = g < gn ? p.q_norm_w : p.k_norm_w;
      float ss = 0.f;
      for (int j = lane; j < d; j += 32) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)d + p.eps);
      for (int j = lane; j < d; j += 32) v[j] = v[j] * r * w[j];
    }
    ATT_SYNC();
  }
  if (p.rope_dim > 0) {
    const float2* tab = (p.rope_table && pos < p.rope_table_len) ? p.rope_table : nullptr;
    for (int g = 0; g < gn; ++g) rope_inplace(q_s[g], p.rope_dim, p.rope_type, pos, p.rope_theta, tab, tid, ATT_THREADS);
    if (owner) rope_inplace(k_s, p.rope_dim, p.rope_type, pos, p.rope_theta, tab, tid, ATT_THREADS);
    ATT_SYNC();
  }
  constexpr int q8 = Q8;                                 // compile-time: the bf16 instantiation carries none of the int8 code
  const int64_t rowb = kv_row_bytes(d, q8);              // bytes per cached row
  float sck = 0.f, scv = 0.f;                            // int8 cache: scales of the new row
  if (q8 && owner) {
    float ak = 0.f, av = 0.f;
    for (int j = tid; j < d; j += ATT_THREADS) { ak = fmaxf(ak, fabsf(k_s[j])); av = fmaxf(av, fabsf(v_s[j])); }
    ak = warp_max(ak); av = warp_max(av);
    if (lane == 0) { qs_s[0][warp] = ak; qs_s[1][warp] = av; }
  }
  if (q8) {
    ATT_SYNC();
    if (owner) {
      for (int w = 0; w < ATT_THREADS / 32; ++w) { sck = fmaxf(sck, qs_s[0][w]); scv = fmaxf(scv, qs_s[1][w]); }
      sck *= 1.f / 127.f; scv *= 1.f / 127.f;
    }
  }
  if (owner && hg == 0) {   // append the new row to the cache (one head group does it)
    const int raw_page = pt[pos / ATT_PAGE], slot = pos % ATT_PAGE;
    const bool page_ok = p.num_pages <= 0 || (unsigned)raw_page < (unsigned)p.num_pages;
    if (!page_ok && tid == 0) atomicExch(&g_attn_decode_error, 3302);
    const int page = page_ok ? raw_page : 0;
    const int64_t rowi = ((int64_t)page * p.n_kv_heads + kvh) * ATT_PAGE + slot;
    if (!page_ok) {
      // a page id outside the cache: nothing is written
    } else if (q8) {
      int8_t* kd = (int8_t*)p.k_cache + rowi * rowb;
      int8_t* vd = (int8_t*)p.v_cache + rowi * rowb;
      for (int j = tid; j < d; j += ATT_THREADS) {
        kd[j] = (int8_t)(sck > 0.f ? fminf(127.f, fmaxf(-127.f, rintf(k_s[j] / sck))) : 0.f);
        vd[j] = (int8_t)(scv > 0.f ? fminf(127.f, fmaxf(-127.f, rintf(v_s[j] / scv))) : 0.f);
      }
      if (tid == 0) { *(float*)(kd + d) = sck; *(float*)(vd + d) = scv; }
    } else {
      const int64_t off = rowi * d;
      for (int j = tid; j < d; j += ATT_THREADS) {
        p.k_cache[off + j] = __float2bfloat16_rn(k_s[j]);
        p.v_cache[off + j] = __float2bfloat16_rn(v_s[j]);
      }
    }
  }
  ATT_SYNC();

  // ---- per-lane query slice: 8 dims, pre-scaled so that exp2 can be used ---------------------
  const int j0 = l16 * 8;
  const bool lane_ok = j0 < d;
  const float qscale = p.scale * 1.4426950408889634f;
  float q[GT][8], acc[GT][8], m[GT], l[GT];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[g][j] = 0.f; q[g][j] = (g < gn && lane_ok) ? q_s[g][j0 + j] * qscale : 0.f; }
  }

  // the owner CTA of a non-zero head group reads the new row from shared memory instead of the
  // cache (another CTA is writing it), everyone else reads the cache only
  // shuffles stay inside a half-warp (all 16 lanes share base / validity), so each half uses its own mask
  const unsigned hmask = 0xFFFFu << (lane & 16);
  // tokens per half-warp per iteration: as many as the registers of this head-group size allow, so that a split of up
  // to 8 * TB tokens (96 for MHA) has all its K/V loads in flight at once and pays the memory latency a single time
  // (DEEP = 0, used when the grid already fills the GPU several times over: 4 tokens, fewer registers, more CTAs per SM)
  constexpr int TB = TBO > 0 ? TBO : DEEP != 1 ? 4 : GT == 1 ? 12 : GT == 2 ? 10 : GT == 4 ? 8 : 4;
  constexpr int TOK_IT = (ATT_THREADS / 16) * TB;
  const int iters = (max(0, end - start) + TOK_IT - 1) / TOK_IT;
  if constexpr (DEEP == 3) {
    static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128 && GT <= 8 && !SUB && Q8 == 0, "tensor-core mode: bf16 cache, head_dim a multiple of 16, up to 8 query heads");
    // head_dim 80: rows of 160 bytes are at most 2-way bank-conflicted unpadded, so whole pages (16 rows, 2560 bytes) are copied
    // with one bulk copy each; the other sizes copy row by row into rows padded by 16 bytes (conflict-free fragment loads)
    constexpr bool PAGE_COPY = HD == 80;
    constexpr int KS = HD / 16, NTL = HD / 8, RS = PAGE_COPY ? 2 * HD : 2 * HD + 16;   // k steps of QK^T, n tiles of PV, row bytes
    constexpr int SLOT = 64 * RS;                                          // 32 K rows, then 32 V rows
    uint8_t* slot = ring + (size_t)warp * SLOT;
    unsigned long long* fb = &sm.full[warp];
    const int gq = lane >> 2, tq = lane & 3;                               // fragment coordinates: row group, thread in group
    if constexpr (!WAITS) {
      if (tid == 0) {
        for (int i = 0; i < ATT_RING; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(att_smem_u32(&sm.full[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      }
      ATT_SYNC();
    }
    auto issue = [&](int it) { att_mma_issue<HD>(p, ring, fb, warp, lane, it, start, end, pt_staged, pt_s, pt, kvh); };
    if (!prefetched && warp < iters) issue(warp);
    // Q fragments (row = query head gq, pre-scaled): a0 = dims 2tq, 2tq+1 of a k step, a2 = the same + 8.  q is split into a
    // bf16 head and a bf16 remainder (two MMAs per tile) so that the scores keep fp32-like precision in q
    uint32_t qa[KS][2], qb[KS][2];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int jq = ks * 16 + 2 * tq + 8 * h;
        const float f0 = gq < gn ? q_s[gq < GT ? gq : 0][jq] * qscale : 0.f, f1 = gq < gn ? q_s[gq < GT ? gq : 0][jq + 1] * qscale : 0.f;
        const uint32_t hi = att_pack_bf16(f0, f1);
        qa[ks][h] = hi;
        qb[ks][h] = att_pack_bf16(f0 - __uint_as_float(hi << 16), f1 - __uint_as_float(hi & 0xFFFF0000u));
      }
    }
    float o[NTL][4];
#pragma unroll
    for (int n = 0; n < NTL; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float mrow = -INFINITY, lsum = 0.f;
    bool stream_ok = true;
    for (int it = warp; it < iters; it += ATT_RING) {
      const int tok0 = start + it * 32;
      const uint32_t parity = (uint32_t)(it / ATT_RING) & 1u;
      bool arrived = false;
      const uint32_t limit = stream_ok ? ATT_WAIT_LIMIT : 1024u;
      for (uint32_t spin = 0; spin < limit; ++spin) if (att_try_wait(fb, parity)) { arrived = true; break; }
      if (!arrived) { stream_ok = false; atomicExch(&g_attn_decode_error, 3201); }
      {   // rows past the end hold stale bytes: zero them; the new token's row comes from the staged k_s / v_s
        const int tok = tok0 + lane;
        uint4* kr4 = (uint4*)(slot + lane * RS); uint4* vr4 = (uint4*)(slot + (32 + lane) * RS);
        if (tok >= end || !stream_ok) {
#pragma unroll
          for (int c = 0; c < HD / 8; ++c) { kr4[c] = make_uint4(0, 0, 0, 0); vr4[c] = make_uint4(0, 0, 0, 0); }
        } else if (owner && tok == pos) {
#pragma unroll
          for (int c = 0; c < HD / 8; ++c) {
            kr4[c] = make_uint4(att_pack_bf16(k_s[8 * c], k_s[8 * c + 1]), att_pack_bf16(k_s[8 * c + 2], k_s[8 * c + 3]),
                                att_pack_bf16(k_s[8 * c + 4], k_s[8 * c + 5]), att_pack_bf16(k_s[8 * c + 6], k_s[8 * c + 7]));
            vr4[c] = make_uint4(att_pack_bf16(v_s[8 * c], v_s[8 * c + 1]), att_pack_bf16(v_s[8 * c + 2], v_s[8 * c + 3]),
                                att_pack_bf16(v_s[8 * c + 4], v_s[8 * c + 5]), att_pack_bf16(v_s[8 * c + 6], v_s[8 * c + 7]));
          }
        }
      }
      __syncwarp();
      // ---- S = Q K^T: 4 tiles of 8 tokens; B fragment = two 4-byte words of the token's K row ----
      float sacc[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const uint8_t* kp = slot + (8 * n + gq) * RS + (ks * 16 + 2 * tq) * 2;
          const uint32_t b0 = *(const uint32_t*)kp, b1 = *(const uint32_t*)(kp + 16);
          att_mma_bf16(sacc[n], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
          att_mma_bf16(sacc[n], qb[ks][0], 0u, qb[ks][1], 0u, b0, b1);
        }
      }
      // ---- online softmax of row gq (the 4 lanes of a group hold its 32 scores) ----
      float mx = -INFINITY;
      bool vis[4][2];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + 8 * n + 2 * tq + e;
          vis[n][e] = tok < end && tok >= lo;
          if (vis[n][e]) mx = fmaxf(mx, sacc[n][e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const float mnew = fmaxf(mrow, mx);
      const float corr = mnew == -INFINITY ? 1.f : exp2f(mrow - mnew);
      uint32_t pa[2][2];
      float psum = 0.f;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const float p0 = vis[n][0] ? exp2f(sacc[n][0] - mnew) : 0.f, p1 = vis[n][1] ? exp2f(sacc[n][1] - mnew) : 0.f;
        const uint32_t pk = att_pack_bf16(p0, p1);
        psum += __uint_as_float(pk << 16) + __uint_as_float(pk & 0xFFFF0000u);      // the rounded values the tensor core multiplies
        pa[n >> 1][n & 1] = pk;
      }
      lsum = lsum * corr + psum;
      mrow = mnew;
#pragma unroll
      for (int n = 0; n < NTL; ++n) { o[n][0] *= corr; o[n][1] *= corr; }
      // ---- O += P V: V rows are [token][dim]; ldmatrix.trans hands out the (token pair, dim) fragments ----
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int n = 0; n < NTL; n += 2) {
          uint32_t r[4];
          const uint8_t* vrow = slot + (32 + 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7)) * RS + (n + (lane >> 4)) * 16;
          att_ldmatrix_x4_trans(r, vrow);
          att_mma_bf16(o[n], pa[kk][0], 0u, pa[kk][1], 0u, r[0], r[1]);
          att_mma_bf16(o[n + 1], pa[kk][0], 0u, pa[kk][1], 0u, r[2], r[3]);
        }
      }
      __syncwarp();
      if (it + ATT_RING < iters) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // this warp's reads of the slot come before the refill
        issue(it + ATT_RING);
      }
    }
    lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, 1);
    lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, 2);
    if (gq < gn) {
#pragma unroll
      for (int n = 0; n < NTL; ++n) { part_s[warp][gq < GT ? gq : 0][8 * n + 2 * tq] = o[n][0]; part_s[warp][gq < GT ? gq : 0][8 * n + 2 * tq + 1] = o[n][1]; }
      if (tq == 0) { part_s[warp][gq < GT ? gq : 0][128] = mrow; part_s[warp][gq < GT ? gq : 0][129] = lsum; }
    }
  } else {
  constexpr bool STREAM = DEEP == 2;
  static_assert(!STREAM || (TB == 4 && !SUB), "streamed mode: 32 tokens (two pages) per iteration, standalone kernel");
  // head groups > 0 of the split that owns the new position read that row from shared memory (only the owner staged it);
  // in streamed mode every owner does: the page copy may race with the append of the new row
  const bool new_from_smem = owner && (STREAM || hg != 0);
  const uint32_t page_bytes = (uint32_t)(ATT_PAGE * rowb), stage_bytes = 4u * page_bytes;     // K page 0, K page 1, V page 0, V page 1
  bool stream_ok = true;
  auto issue = [&](int it) {                               // thread 0: request the two pages of iteration `it`
    const int slot = it % ATT_RING;
    const int tok0 = start + it * TOK_IT;
    const int np = min(2, (end - tok0 + ATT_PAGE - 1) / ATT_PAGE);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(&sm.full[slot])), "r"(2u * np * page_bytes) : "memory");
    for (int pi = 0; pi < np; ++pi) {
      const int tk = tok0 + pi * ATT_PAGE;
      const int page = pt_staged ? pt_s[(tk - start) / ATT_PAGE] : att_page(p, pt[tk / ATT_PAGE]);
      const int64_t boff = ((int64_t)page * p.n_kv_heads + kvh) * ATT_PAGE * rowb;
      uint8_t* dst = ring + (size_t)slot * stage_bytes + (size_t)pi * page_bytes;
      att_bulk_g2s(dst, (const uint8_t*)p.k_cache + boff, page_bytes, &sm.full[slot]);
      att_bulk_g2s(dst + 2 * page_bytes, (const uint8_t*)p.v_cache + boff, page_bytes, &sm.full[slot]);
    }
  };
  if (STREAM) {
    if (tid == 0) {
      for (int i = 0; i < ATT_RING; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(att_smem_u32(&sm.full[i])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      for (int it = 0; it < min(ATT_RING, iters); ++it) issue(it);
    }
    ATT_SYNC();
  }
  for (int it = 0; it < iters; ++it) {
    const int base = start + (it * (ATT_THREADS / 16) + hw) * TB;
    uint4 kr[TB], vr[TB];
    if (STREAM) {
      unsigned long long* fb = &sm.full[it % ATT_RING];
      const uint32_t parity = (uint32_t)(it / ATT_RING) & 1u;
      bool arrived = false;
      const uint32_t limit = stream_ok ? ATT_WAIT_LIMIT : 1024u;       // after a failure the remaining stages get a short wait each
      for (uint32_t spin = 0; spin < limit; ++spin) if (att_try_wait(fb, parity)) { arrived = true; break; }
      if (!arrived) { stream_ok = false; atomicExch(&g_attn_decode_error, 3201); }
      const uint8_t* st = ring + (size_t)(it % ATT_RING) * stage_bytes + (size_t)(hw >> 2) * page_bytes;      // my page of the stage
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        const int tok = base + t;
        const bool okl = stream_ok && lane_ok && tok < end && !(new_from_smem && tok == pos);
        const uint8_t* kp = st + (size_t)((hw & 3) * TB + t) * rowb;
        const uint8_t* vp = kp + 2 * page_bytes;
        if (q8) {
          const uint2 kc = okl ? *(const uint2*)(kp + j0) : make_uint2(0, 0);
          const uint2 vc = okl ? *(const uint2*)(vp + j0) : make_uint2(0, 0);
          kr[t] = make_uint4(kc.x, kc.y, okl ? *(const uint32_t*)(kp + d) : 0u, 0u);
          vr[t] = make_uint4(vc.x, vc.y, okl ? *(const uint32_t*)(vp + d) : 0u, 0u);
        } else {
          kr[t] = okl ? *(const uint4*)(kp + 2 * j0) : make_uint4(0, 0, 0, 0);
          vr[t] = okl ? *(const uint4*)(vp + 2 * j0) : make_uint4(0, 0, 0, 0);
        }
      }
      ATT_SYNC();                                          // every thread has taken its rows: the stage may be refilled
      if (tid == 0 && it + ATT_RING < iters) issue(it + ATT_RING);
    } else {
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int tok = base + t;
      const bool okl = lane_ok && tok < end && !(new_from_smem && tok == pos);
      const int tk = min(tok, end - 1 > start ? end - 1 : start);
      const int page = pt_staged ? pt_s[(tk - start) / ATT_PAGE] : att_page(p, pt[tk / ATT_PAGE]);
      const int64_t rowi = ((int64_t)page * p.n_kv_heads + kvh) * ATT_PAGE + (tk % ATT_PAGE);
      if (q8) {                                           // 8 codes (x, y) and the row scale (z)
        const uint8_t* kp = (const uint8_t*)p.k_cache + rowi * rowb;
        const uint8_t* vp = (const uint8_t*)p.v_cache + rowi * rowb;
        const uint2 kc = okl ? *(const uint2*)(kp + j0) : make_uint2(0x80808080u ^ 0x80808080u, 0);
        const uint2 vc = okl ? *(const uint2*)(vp + j0) : make_uint2(0, 0);
        kr[t] = make_uint4(kc.x, kc.y, okl ? *(const uint32_t*)(kp + d) : 0u, 0u);
        vr[t] = make_uint4(vc.x, vc.y, okl ? *(const uint32_t*)(vp + d) : 0u, 0u);
      } else {
        const int64_t off = rowi * d + j0;
        kr[t] = okl ? *(const uint4*)(p.k_cache + off) : make_uint4(0, 0, 0, 0);
        vr[t] = okl ? *(const uint4*)(p.v_cache + off) : make_uint4(0, 0, 0, 0);
      }
    }
    }
    float sc[GT][TB];
    // pass 1: scores (K converted one token at a time)
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      float kf[8];
      if (q8) {
        const float sc = __uint_as_float(kr[t].z);
        q8_word_to_float(kr[t].x, sc, kf); q8_word_to_float(kr[t].y, sc, kf + 4);
      } else {
        const uint32_t kw[4] = {kr[t].x, kr[t].y, kr[t].z, kr[t].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { kf[2 * j] = __uint_as_float(kw[j] << 16); kf[2 * j + 1] = __uint_as_float(kw[j] & 0xFFFF0000u); }
      }
      if (new_from_smem && base + t == pos && lane_ok) {   // new row straight from shared memory (rounded like the cache)
#pragma unroll
        for (int j = 0; j < 8; ++j) kf[j] = q8 ? q8_round(k_s[j0 + j], sck) : __bfloat162float(__float2bfloat16_rn(k_s[j0 + j]));
      }
      const bool valid = base + t < end && base + t >= lo;
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float x = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) x += q[g][j] * kf[j];
        x += __shfl_xor_sync(hmask, x, 8);
        x += __shfl_xor_sync(hmask, x, 4);
        x += __shfl_xor_sync(hmask, x, 2);
        x += __shfl_xor_sync(hmask, x, 1);
        sc[g][t] = valid ? x : -INFINITY;
      }
    }
    // running max / rescale per head, scores -> probabilities
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float mn = m[g];
#pragma unroll
      for (int t = 0; t < TB; ++t) mn = fmaxf(mn, sc[g][t]);
      const bool none = mn == -INFINITY;       // nothing valid seen yet by this stream
      const float corr = none ? 1.f : exp2f(m[g] - mn);     // m = -inf on the first valid pass -> 0
      l[g] *= corr;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] *= corr;
#pragma unroll
      for (int t = 0; t < TB; ++t) { sc[g][t] = none ? 0.f : exp2f(sc[g][t] - mn); l[g] += sc[g][t]; }
      m[g] = mn;
    }
    // pass 2: weighted values (V converted one token at a time)
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      float vf[8];
      if (q8) {
        const float sc = __uint_as_float(vr[t].z);
        q8_word_to_float(vr[t].x, sc, vf); q8_word_to_float(vr[t].y, sc, vf + 4);
      } else {
        const uint32_t vw[4] = {vr[t].x, vr[t].y, vr[t].z, vr[t].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { vf[2 * j] = __uint_as_float(vw[j] << 16); vf[2 * j + 1] = __uint_as_float(vw[j] & 0xFFFF0000u); }
      }
      if (new_from_smem && base + t == pos && lane_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) vf[j] = q8 ? q8_round(v_s[j0 + j], scv) : __bfloat162float(__float2bfloat16_rn(v_s[j0 + j]));
      }
#pragma unroll
      for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] += sc[g][t] * vf[j];
    }
  }

  // ---- combine: the two half-warps of a warp through shuffles, then the warps through shared memory ----
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const float mo = __shfl_xor_sync(0xFFFFFFFFu, m[g], 16), lo2 = __shfl_xor_sync(0xFFFFFFFFu, l[g], 16);
    const float mm = fmaxf(m[g], mo);
    const float c0 = m[g] == -INFINITY ? 0.f : exp2f(m[g] - mm), c1 = mo == -INFINITY ? 0.f : exp2f(mo - mm);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float ao = __shfl_xor_sync(0xFFFFFFFFu, acc[g][j], 16);
      acc[g][j] = c0 * acc[g][j] + c1 * ao;
    }
    l[g] = c0 * l[g] + c1 * lo2;
    m[g] = mm;
  }
  // ---- combine the 8 half-warp streams of this CTA -------------------------------------------
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (g < gn && lane < 16) {
      if (lane_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) part_s[warp][g][j0 + j] = acc[g][j];
      }
      if (lane == 0) { part_s[warp][g][128] = m[g]; part_s[warp][g][129] = l[g]; }
    }
  }
  }
  ATT_SYNC();
  const int S = p.splits;
  float* push_dst = nullptr;                              // (push mode) this split's slot in rank 0's gather buffer
  if (PUSH) {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");               // phase 1 complete: every CTA of the cluster is running
    push_dst = cg::this_cluster().map_shared_rank(&gat_s[0][0][0], 0) + (int64_t)split * GT * 130;
  }
  for (int i = tid; i < gn * d + gn; i += ATT_THREADS) {
    const bool stat = i >= gn * d;                 // the trailing gn items carry (max, sum) of each head
    const int g = stat ? i - gn * d : i / d, j = stat ? 0 : i - g * d;
    float mm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, part_s[w][g][128]);
    float a = 0.f, ll = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float mw = part_s[w][g][128];
      const float c = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      a += c * part_s[w][g][j]; ll += c * part_s[w][g][129];
    }
    if (MERGE == MERGE_NONE) {
      if (!stat) p.out[(int64_t)b * p.ld_out + (kvh * G + g0 + g) * d + j] = a / ll;
    } else if (MERGE == MERGE_CLUSTER) {
      if (PUSH) {                                          // straight into rank 0's shared memory
        if (stat) { push_dst[g * 130 + 128] = mm; push_dst[g * 130 + 129] = ll; } else push_dst[g * 130 + j] = a;
      } else {
        if (stat) { res_s[g][128] = mm; res_s[g][129] = ll; } else res_s[g][j] = a;
      }
    } else {
      float* dst = p.partial + (((int64_t)b * p.n_heads + kvh * G + g0 + g) * S + split) * (d + 2);
      if (stat) { dst[d] = mm; dst[d + 1] = ll; } else dst[j] = a;
    }
  }
  if (MERGE == MERGE_NONE) return;

  if (MERGE == MERGE_CLUSTER && PUSH) {
    // ---- every split stores its result into rank 0's gather buffer, signals, and leaves; rank 0 merges locally ----
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");             // phase 2: my stores are done
    if (cg::this_cluster().block_rank() != 0) return;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    for (int i = tid; i < gn * d; i += ATT_THREADS) {
      const int g = i / d, j = i - g * d;
      float mm = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < ATT_MAX_CLUSTER; ++sp) if (sp < S) mm = fmaxf(mm, gat_s[sp][g][128]);
      float a = 0.f, ll = 0.f;
#pragma unroll
      for (int sp = 0; sp < ATT_MAX_CLUSTER; ++sp) {
        if (sp < S) {
          const float ms = gat_s[sp][g][128];
          const float c = ms == -INFINITY ? 0.f : exp2f(ms - mm);
          a += c * gat_s[sp][g][j]; ll += c * gat_s[sp][g][129];
        }
      }
      p.out[(int64_t)b * p.ld_out + (kvh * G + g0 + g) * d + j] = a / ll;
    }
    return;
  }
  if (MERGE == MERGE_CLUSTER) {
    // ---- (8 heads per CTA) cluster rank 0 merges the splits out of its peers' shared memory ----------------------
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                  // every CTA's res_s is complete and visible
    if (cluster.block_rank() == 0) {
      // the loops over the splits are unrolled to the cluster size so that the remote loads are independent and in flight together
      for (int i = tid; i < gn * d; i += ATT_THREADS) {
        const int g = i / d, j = i - g * d;
        float ms[ATT_MAX_CLUSTER], av[ATT_MAX_CLUSTER], lv[ATT_MAX_CLUSTER];
#pragma unroll
        for (int sp = 0; sp < ATT_MAX_CLUSTER; ++sp) {
          const float* r = cluster.map_shared_rank(&res_s[0][0], sp < S ? sp : 0) + g * 130;
          ms[sp] = sp < S ? r[128] : -INFINITY; av[sp] = r[j]; lv[sp] = r[129];
        }
        float mm = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < ATT_MAX_CLUSTER; ++sp) mm = fmaxf(mm, ms[sp]);
        float a = 0.f, ll = 0.f;
#pragma unroll
        for (int sp = 0; sp < ATT_MAX_CLUSTER; ++sp) {
          const float c = ms[sp] == -INFINITY ? 0.f : exp2f(ms[sp] - mm);
          a += c * av[sp]; ll += c * lv[sp];
        }
        p.out[(int64_t)b * p.ld_out + (kvh * G + g0 + g) * d + j] = a / ll;
      }
    }
    cluster.sync();                                  // peers keep their shared memory alive until rank 0 has read it
    return;
  }

  // ---- last CTA of this (sequence, kv head, head group) merges the splits ----------------------
  __threadfence();
  ATT_SYNC();
  int32_t* ctr = p.counters + (int64_t)b * (p.n_kv_heads * hgroups) + bx;
  if (tid == 0) {
    const int ticket = atomicAdd(ctr, 1);
    last_flag = ticket == S - 1;
    if (last_flag) *ctr = 0;       // self-cleaning for the next launch
  }
  ATT_SYNC();
  if (!last_flag) return;
  __threadfence();
  for (int i = tid; i < gn * d; i += ATT_THREADS) {
    const int g = i / d, j = i - g * d;
    const float* src = p.partial + ((int64_t)b * p.n_heads + kvh * G + g0 + g) * S * (d + 2);
    float mm = -INFINITY;
    for (int s = 0; s < S; ++s) mm = fmaxf(mm, __ldcg(src + (int64_t)s * (d + 2) + d));
    float a = 0.f, ll = 0.f;
    for (int s = 0; s < S; ++s) {
      const float ms = __ldcg(src + (int64_t)s * (d + 2) + d);
      const float c = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      a += c * __ldcg(src + (int64_t)s * (d + 2) + j);
      ll += c * __ldcg(src + (int64_t)s * (d + 2) + d + 1);
    }
    p.out[(int64_t)b * p.ld_out + (kvh * G + g0 + g) * d + j] = a / ll;
  }
}
#undef ATT_SYNC

}  // namespace rlz
