// Token selection on the GPU: greedy argmax, and temperature / top-k / top-p / min-p sampling
// with an exact radix select, plus repetition / presence / frequency penalties.  One CTA per
// sequence; per-sequence parameters come from device arrays so a continuous batch can mix
// greedy and sampled requests in one launch.
//
// The reference picks greedy tokens with argmax_block_reduce/final_reduce and downloads the
// logits for anything else (src/cuda/executor/layers/par-062.rs:124-330,
// src/gguf/cuda/generate_2.rs:526-533); the sampling order (penalties -> temperature -> top-k
// -> top-p) follows its CPU sampler (src/gguf/inference/fails.rs:92-336).
#include "common.cuh"
#include "gemv_params.h"
#include <math.h>

namespace rlz {

constexpr int SAMP_THREADS = 1024;
constexpr int SAMP_MAX_CAND = 1024;

__device__ __forceinline__ uint32_t float_key(float x) {      // order-preserving map to uint
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// (max value, smallest index attaining it) over the block; result valid in all threads
__device__ void block_argmax(float v, int idx, float* sval, int* sidx, float* out_v, int* out_i) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { sval[warp] = v; sidx[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    v = lane < nw ? sval[lane] : -INFINITY; idx = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (lane == 0) { sval[32] = v; sidx[32] = idx; }
  }
  __syncthreads();
  *out_v = sval[32]; *out_i = sidx[32];
}

__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* logits, int64_t ld, int vocab, int32_t* out, float* out_val,
                                                              int index_offset) {
  __shared__ float sval[33]; __shared__ int sidx[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (int64_t)blockIdx.x * ld;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float v = row[i]; if (v > best) { best = v; bi = i; } }
  float v; int i;
  block_argmax(best, bi, sval, sidx, &v, &i);
  if (threadIdx.x == 0) { out[blockIdx.x] = i + index_offset; if (out_val) out_val[blockIdx.x] = v; }
}

// Multi-CTA argmax: grid (rows, slices).  Every CTA reduces its slice of the row, folds (value, smallest index) into a
// 64-bit key with atomicMax, and the last CTA of the row to finish (ticket counter) decodes the key, writes the result
// and leaves key and counter zeroed for the next launch (the scratch is a file-scope device array, self-cleaning).
constexpr int ARGMAX_MAX_ROWS = 4096;
__device__ unsigned long long g_argmax_key[ARGMAX_MAX_ROWS];
__device__ unsigned int g_argmax_cnt[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(SAMP_THREADS) argmax_sliced_kernel(const float* logits, int64_t ld, int vocab, int32_t* out, float* out_val,
                                                                     int index_offset) {
  __shared__ float sval[33]; __shared__ int sidx[33];
  __shared__ int last_s;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, nsl = gridDim.y;
  const float* row = logits + (int64_t)r * ld;
  const int per = ((vocab + nsl - 1) / nsl + 3) & ~3;
  const int i0 = blockIdx.y * per, i1 = min(vocab, i0 + per);
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) { const float v = row[i]; if (v > best) { best = v; bi = i; } }
  float v; int i;
  block_argmax(best, bi, sval, sidx, &v, &i);
  if (threadIdx.x == 0) {
    if (i != 0x7fffffff) atomicMax(&g_argmax_key[r], ((unsigned long long)float_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i));
    __threadfence();
    last_s = atomicAdd(&g_argmax_cnt[r], 1u) == (unsigned)nsl - 1;
  }
  __syncthreads();
  if (!last_s || threadIdx.x != 0) return;
  __threadfence();
  const unsigned long long key = atomicExch(&g_argmax_key[r], 0ull);
  g_argmax_cnt[r] = 0;
  const uint32_t kv = (uint32_t)(key >> 32), idx = 0xFFFFFFFFu - (uint32_t)key;
  out[r] = (key ? (int)idx : 0) + index_offset;
  if (out_val) out_val[r] = key ? __uint_as_float((kv & 0x80000000u) ? (kv & 0x7FFFFFFFu) : ~kv) : -INFINITY;
}

struct SampleParams {
  const float* logits; int64_t ld; int32_t vocab; int32_t batch;
  const float* temperature;   // [B]; <= 0 -> greedy
  const int32_t* top_k;       // [B]; <= 0 -> candidate cap (1024)
  const float* top_p;         // [B]; >= 1 -> off
  const float* min_p;         // [B] or null
  const float* uniform;       // [B] in [0,1)
  int32_t* out;               // [B]
  float* out_logprob;         // [B] or null: log-probability of the chosen token under the filtered distribution
};

// Shared-memory state of one row's selection
struct SampleSmem {
  float sval[33]; int sidx[33];
  unsigned hist[256];
  float cval[SAMP_MAX_CAND]; int cidx[SAMP_MAX_CAND];
  float csum[SAMP_MAX_CAND];
  unsigned prefix, kk, count, ties;
  int pick;
};

// Where a row's values come from: the logits of a vocabulary slice (token id = position + offset)
struct RowSrc {
  const float* row; int off;
  __device__ __forceinline__ float value(int i) const { return row[i]; }
  __device__ __forceinline__ int token(int i) const { return i + off; }
};
// (the gathered candidate lists of a vocabulary-sharded head are the other source, see sample_merge_kernel)

// Largest value of the row (ties: smallest token id), valid in all threads
template <class Src>
__device__ __forceinline__ void row_argmax(SampleSmem& S, const Src& src, int V, float* vmax, int* tmax) {
  float best = -INFINITY; int bt = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
    const float v = src.value(i); const int t = src.token(i);
    if (v > best || (v == best && t < bt)) { best = v; bt = t; }
  }
  block_argmax(best, bt, S.sval, S.sidx, vmax, tmax);
}

// The k largest values of the row (exact k-th key by 4 x 8-bit radix select) into S.cval / S.cidx (token ids), unsorted, padded
// with -inf up to SAMP_MAX_CAND; returns how many were taken
template <class Src>
__device__ __forceinline__ int select_topk(SampleSmem& S, const Src& src, int V, int k) {
  const int tid = threadIdx.x;
  if (tid == 0) { S.prefix = 0; S.kk = (unsigned)k; }
  for (int round = 0; round < 4; ++round) {
    const int shift = 24 - 8 * round;
    if (tid < 256) S.hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = S.prefix, pmask = round == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += SAMP_THREADS) {
      const uint32_t key = float_key(src.value(i));
      if ((key & pmask) == prefix) atomicAdd(&S.hist[(key >> shift) & 0xFFu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned cum = 0, kk = S.kk; int bin = 255;
      for (; bin > 0; --bin) { if (cum + S.hist[bin] >= kk) break; cum += S.hist[bin]; }
      S.kk = kk - cum;                        // still needed from inside this bin
      S.prefix = prefix | ((unsigned)bin << shift);
    }
    __syncthreads();
  }
  const uint32_t tkey = S.prefix;             // key of the k-th largest value
  const unsigned ties_wanted = S.kk;          // how many elements equal to it belong to the top k
  if (tid == 0) { S.count = 0; S.ties = 0; }
  for (int i = tid; i < SAMP_MAX_CAND; i += SAMP_THREADS) { S.cval[i] = -INFINITY; S.cidx[i] = 0x7fffffff; }
  __syncthreads();
  for (int i = tid; i < V; i += SAMP_THREADS) {
    const float v = src.value(i); const uint32_t key = float_key(v);
    bool take = key > tkey;
    if (key == tkey) take = atomicAdd(&S.ties, 1u) < ties_wanted;
    if (take) { const unsigned slot = atomicAdd(&S.count, 1u); if (slot < SAMP_MAX_CAND) { S.cval[slot] = v; S.cidx[slot] = src.token(i); } }
  }
  __syncthreads();
  return (int)min(S.count, (unsigned)SAMP_MAX_CAND);
}

// Candidates in S.cval / S.cidx (n valid): sort by (value descending, token id ascending), softmax with temperature relative to
// vmax, min-p / top-p filtering, inverse-CDF draw with p.uniform[b]; writes p.out[b]
__device__ __forceinline__ void sort_and_draw(SampleSmem& S, const SampleParams& p, int b, int n, float vmax, float temp) {
  const int tid = threadIdx.x;
  float* cval = S.cval; int* cidx = S.cidx; float* csum = S.csum;
  for (int size = 2; size <= SAMP_MAX_CAND; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i) {
        const bool desc = (i & size) == 0;
        const float vi = cval[i], vj = cval[j]; const int ii = cidx[i], ij = cidx[j];
        const bool i_first = vi > vj || (vi == vj && ii < ij);      // i should precede j in descending order
        if (desc ? !i_first : i_first) { cval[i] = vj; cval[j] = vi; cidx[i] = ij; cidx[j] = ii; }
      }
      __syncthreads();
    }
  }
  const float inv_t = 1.f / temp;
  float pr = tid < n ? __expf((cval[tid] - vmax) * inv_t) : 0.f;
  if (p.min_p && p.min_p[b] > 0.f && pr < p.min_p[b]) pr = 0.f;      // relative to the top probability (= 1 here)
  csum[tid] = pr;
  __syncthreads();
  for (int off = 1; off < SAMP_MAX_CAND; off <<= 1) {                // inclusive scan
    const float add = tid >= off ? csum[tid - off] : 0.f;
    __syncthreads();
    csum[tid] += add;
    __syncthreads();
  }
  const float total = csum[SAMP_MAX_CAND - 1];
  const float top_p = p.top_p[b];
  if (tid == 0) S.pick = n - 1;
  __syncthreads();
  // nucleus: smallest prefix whose mass reaches top_p * total
  float kept = total;
  if (top_p < 1.f) {
    const float need = top_p * total;
    const bool here = csum[tid] >= need && (tid == 0 || csum[tid - 1] < need);
    if (here) S.pick = tid;
    __syncthreads();
    kept = csum[S.pick];
    __syncthreads();
  }
  const int last = top_p < 1.f ? S.pick : n - 1;
  const float target = p.uniform[b] * kept;
  if (tid == 0) S.pick = last;
  __syncthreads();
  if (tid <= last && csum[tid] > target && (tid == 0 || csum[tid - 1] <= target)) S.pick = tid;
  __syncthreads();
  if (tid == 0) {
    const int c = S.pick;
    p.out[b] = cidx[c];
    if (p.out_logprob) { const float pc = c == 0 ? csum[0] : csum[c] - csum[c - 1]; p.out_logprob[b] = logf(fmaxf(pc, 1e-30f) / kept); }
  }
}

__device__ __forceinline__ int clamp_k(int k, int V) {
  if (k <= 0 || k > SAMP_MAX_CAND) k = SAMP_MAX_CAND;
  return k > V ? V : k;
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(const __grid_constant__ SampleParams p) {
  __shared__ SampleSmem S;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const RowSrc src{p.logits + (int64_t)b * p.ld, 0};
  const float temp = p.temperature[b];
  const int k = p.top_k[b];
  float vmax; int tmax;
  row_argmax(S, src, p.vocab, &vmax, &tmax);
  if (temp <= 0.f || k == 1) { if (threadIdx.x == 0) { p.out[b] = tmax; if (p.out_logprob) p.out_logprob[b] = 0.f; } return; }
  const int n = select_topk(S, src, p.vocab, clamp_k(k, p.vocab));
  sort_and_draw(S, p, b, n, vmax, temp);
}

// ---- vocabulary-sharded heads: per-rank candidates, exchange over peer memory, identical draw on every rank -----------------
// Every rank selects the top-k of ITS vocabulary slice (the global top-k is contained in the union of the local ones), stores
// the (value, token id) pairs into every rank's inbox and publishes one flag word per (rank, row): (epoch << 11) | count.  The
// second kernel waits (bounded) for the world's flags of its row and runs the same selection and draw over the gathered
// candidates; with the same uniform number every rank picks the same token.  Replaces an all-gather of the whole vocabulary row.
struct ShardSample {
  uint2* inbox[GEMV_AR_MAX_RANKS];       // rank r's candidate inbox: [parity 2][world][batch_cap][K] pairs
  uint32_t* flags[GEMV_AR_MAX_RANKS];    // rank r's flags: [parity 2][world][batch_cap]
  const uint32_t* epoch; int32_t* status;
  int64_t spin_limit;
  int32_t rank, world, batch_cap, K;     // K <= SAMP_MAX_CAND pairs reserved per (rank, row)
  int32_t index_offset, _pad;            // first token id of this rank's slice
};

// one row's candidate lists as they lie in an inbox: writer r's list starts r * stride pairs on, its first cnt[r] pairs are valid
struct Gathered {
  const uint2* base; const int* cnt; int K; int64_t stride;
  __device__ __forceinline__ float value(int i) const { const int r = i / K, j = i - r * K; return j < cnt[r] ? __uint_as_float(base[r * stride + j].x) : -INFINITY; }
  __device__ __forceinline__ int token(int i) const { const int r = i / K, j = i - r * K; return j < cnt[r] ? (int)base[r * stride + j].y : 0x7fffffff; }
};

__global__ void __launch_bounds__(SAMP_THREADS) sample_push_kernel(const __grid_constant__ SampleParams p, const __grid_constant__ ShardSample c) {
  __shared__ SampleSmem S;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const RowSrc src{p.logits + (int64_t)b * p.ld, c.index_offset};
  const float temp = p.temperature[b];
  int k = p.top_k[b];
  int n;
  if (temp <= 0.f || k == 1) {                             // greedy rows exchange one candidate
    float vmax; int tmax;
    row_argmax(S, src, p.vocab, &vmax, &tmax);
    if (tid == 0) { S.cval[0] = vmax; S.cidx[0] = tmax; }
    __syncthreads();
    n = 1;
  } else {
    k = clamp_k(k, p.vocab);
    n = select_topk(S, src, p.vocab, k > c.K ? c.K : k);
  }
  const uint32_t epoch = *c.epoch;
  const int64_t slot = ((int64_t)(epoch & 1u) * c.world + c.rank) * c.batch_cap + b;
  for (int q = 0; q < c.world; ++q) {
    uint2* dst = c.inbox[q] + slot * c.K;
    for (int i = tid; i < n; i += SAMP_THREADS) dst[i] = make_uint2(__float_as_uint(S.cval[i]), (uint32_t)S.cidx[i]);
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world) {
    const uint32_t word = ((epoch & 0x1FFFFFu) << 11) | (uint32_t)n;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(c.flags[tid] + slot), "r"(word) : "memory");
  }
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_merge_kernel(const __grid_constant__ SampleParams p, const __grid_constant__ ShardSample c) {
  __shared__ SampleSmem S;
  __shared__ int cnt[GEMV_AR_MAX_RANKS];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const uint32_t epoch = *c.epoch;
  const int64_t base = (int64_t)(epoch & 1u) * c.world * c.batch_cap;
  if (tid < c.world) {                                     // one poller per writer; a wait that runs out leaves that writer's list empty
    const uint32_t* f = c.flags[c.rank] + base + (int64_t)tid * c.batch_cap + b;
    int got = -1;
    for (int64_t spins = 0; spins <= c.spin_limit; ++spins) {
      uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((v >> 11) == (epoch & 0x1FFFFFu)) { got = (int)(v & 0x7FFu); break; }
    }
    if (got < 0) { atomicExch(c.status, 2006); got = 0; }
    cnt[tid] = got > c.K ? c.K : got;
  }
  __syncthreads();
  // row b of every writer, as one [world][K] array: the writers' slots of a row are batch_cap * K pairs apart
  const uint2* mine = c.inbox[c.rank] + (base + b) * c.K;
  const Gathered src{mine, cnt, c.K, (int64_t)c.batch_cap * c.K};
  const int V = c.world * c.K;
  const float temp = p.temperature[b];
  const int k = p.top_k[b];
  float vmax; int tmax;
  row_argmax(S, src, V, &vmax, &tmax);
  if (temp <= 0.f || k == 1) { if (tid == 0) { p.out[b] = tmax; if (p.out_logprob) p.out_logprob[b] = 0.f; } return; }
  int total = 0;
  for (int r = 0; r < c.world; ++r) total += cnt[r];
  int kk = clamp_k(k, total < 1 ? 1 : total);
  if (kk > c.K) kk = c.K;                                  // beyond K per rank the union of the lists is no longer the global top
  const int n = select_topk(S, src, V, kk);
  sort_and_draw(S, p, b, n, vmax, temp);
}

// logits[b, tok] adjusted for every distinct token in history[b, :] (entries < 0 are padding):
// repetition penalty (divide positive / multiply negative), presence and frequency penalties.
__global__ void penalties_kernel(float* logits, int64_t ld, int vocab, const int32_t* history, int window,
                                 const float* repetition, const float* presence, const float* frequency) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int32_t* h = history + (int64_t)b * window;
  const float rep = repetition ? repetition[b] : 1.f, pres = presence ? presence[b] : 0.f, freq = frequency ? frequency[b] : 0.f;
  if (rep == 1.f && pres == 0.f && freq == 0.f) return;
  for (int i = threadIdx.x; i < window; i += blockDim.x) {
    const int tok = h[i];
    if (tok < 0 || tok >= vocab) continue;
    int count = 0; bool first = true;
    for (int j = 0; j < window; ++j) if (h[j] == tok) { ++count; if (j < i) first = false; }
    if (!first) continue;
    float v = logits[(int64_t)b * ld + tok];
    if (rep != 1.f) v = v > 0.f ? v / rep : v * rep;
    v -= pres + freq * (float)count;
    logits[(int64_t)b * ld + tok] = v;
  }
}

// The token fed at this step joins the sequence's history ring (what the penalties look at): history[b, position % window] = token.
__global__ void history_push_kernel(int32_t* history, int window, const int32_t* tokens, const int32_t* positions, int batch) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch && positions[b] >= 0) history[(int64_t)b * window + positions[b] % window] = tokens[b];
}

// Per-sequence logit controls applied in place before the sampling kernel, one CTA per row:
//   * an additive row (`bias`, used for OpenAI-style logit_bias and, with -inf entries, for grammar / tool-call token masks)
//     for the rows whose `bias_on` flag is set;
//   * repetition / presence / frequency penalties over the distinct tokens of the history ring.
// `index_offset` / `vocab` describe the slice of the vocabulary held in `logits` (vocabulary-sharded heads); bias rows hold
// the same slice.  Replaces the host-side LogitProcessorChain of the reference (src/generate/mod.rs:107-400).
__global__ void __launch_bounds__(SAMP_THREADS) logit_controls_kernel(float* logits, int64_t ld, int vocab, int index_offset, const int32_t* history,
                                                                      int window, const float* repetition, const float* presence, const float* frequency,
                                                                      const float* bias, int64_t ld_bias, const int32_t* bias_on) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  float* row = logits + (int64_t)b * ld;
  if (bias && bias_on && bias_on[b]) {
    const float* br = bias + (int64_t)b * ld_bias;
    for (int i = threadIdx.x; i < vocab; i += SAMP_THREADS) row[i] += br[i];
    __syncthreads();
  }
  const float rep = repetition ? repetition[b] : 1.f, pres = presence ? presence[b] : 0.f, freq = frequency ? frequency[b] : 0.f;
  if (!history || (rep == 1.f && pres == 0.f && freq == 0.f)) return;
  const int32_t* h = history + (int64_t)b * window;
  for (int i = threadIdx.x; i < window; i += SAMP_THREADS) {
    const int tok = h[i];
    if (tok < index_offset || tok >= index_offset + vocab) continue;
    int count = 0; bool first = true;
    for (int j = 0; j < window; ++j) if (h[j] == tok) { ++count; if (j < i) first = false; }
    if (!first) continue;
    float v = row[tok - index_offset];
    if (rep != 1.f) v = v > 0.f ? v / rep : v * rep;
    v -= pres + freq * (float)count;
    row[tok - index_offset] = v;
  }
}

// Scoring: per row, the pieces of log softmax(logits)[target] over this rank's vocabulary slice [index_offset, index_offset + vocab):
// out[row] = {max, sum exp(logit - max), logit of the target if it lies in the slice else -inf}.  With one slice the log-probability
// is out[2] - out[0] - log(out[1]); vocabulary-sharded heads combine the triples of all ranks first.  One CTA per row, one pass for
// the maximum and one for the sum (the row stays in L2 between them).  Replaces the reference's host-side log-softmax over
// downloaded logits (src/gguf/cuda/generate_2.rs:590-780).
__global__ void __launch_bounds__(SAMP_THREADS) logprob_rows_kernel(const float* logits, int64_t ld, int vocab, const int32_t* targets, int index_offset,
                                                                    float* out) {
  __shared__ float red[40];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (int64_t)row * ld;
  float m = -INFINITY;
  for (int i = tid; i < vocab; i += SAMP_THREADS) m = fmaxf(m, l[i]);
  m = block_max(m, red);
  float s = 0.f;
  for (int i = tid; i < vocab; i += SAMP_THREADS) s += __expf(l[i] - m);
  s = block_sum(s, red);
  if (tid == 0) {
    const int t = targets[row] - index_offset;
    out[3 * row + 0] = m;
    out[3 * row + 1] = s;
    out[3 * row + 2] = (t >= 0 && t < vocab) ? l[t] : -INFINITY;
  }
}

}  // namespace rlz

extern "C" {
using namespace rlz;

int rlz_history_push(int32_t* history, int window, const int32_t* tokens, const int32_t* positions, int batch, void* stream) {
  if (window < 1 || batch < 1) return -1;
  return (int)launch(history_push_kernel, dim3((batch + 63) / 64), dim3(64), 0, (cudaStream_t)stream, history, window, tokens, positions, batch);
}

int rlz_logit_controls(float* logits, long long ld, int vocab, int index_offset, int batch, const int32_t* history, int window, const float* repetition,
                       const float* presence, const float* frequency, const float* bias, long long ld_bias, const int32_t* bias_on, void* stream) {
  if (vocab < 1 || batch < 1) return -1;
  return (int)launch(logit_controls_kernel, dim3(batch), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, logits, (int64_t)ld, vocab, index_offset, history,
                     window, repetition, presence, frequency, bias, (int64_t)ld_bias, bias_on);
}

int rlz_logprob_rows(const float* logits, long long ld, int vocab, int rows, const int32_t* targets, int index_offset, float* out, void* stream) {
  if (vocab < 1 || rows < 1) return -1;
  return (int)launch(logprob_rows_kernel, dim3(rows), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, logits, (int64_t)ld, vocab, targets, index_offset, out);
}

int rlz_argmax(const float* logits, long long ld, int vocab, int batch, int32_t* out, float* out_val, int index_offset, void* stream) {
  if (vocab < 1 || batch < 1) return -1;
  // wide rows and few sequences: split every row over several CTAs (one CTA per row leaves the GPU idle)
  const int slices = vocab >= 16384 && batch <= ARGMAX_MAX_ROWS ? (batch >= 64 ? 4 : vocab / 4096 > 32 ? 32 : vocab / 4096) : 1;
  if (slices > 1)
    return (int)launch(argmax_sliced_kernel, dim3(batch, slices), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, logits, (int64_t)ld, vocab, out, out_val,
                       index_offset);
  return (int)launch(argmax_kernel, dim3(batch), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, logits, (int64_t)ld, vocab, out, out_val, index_offset);
}

int rlz_sample(const SampleParams* p, void* stream) {
  if (p->vocab < 1 || p->batch < 1) return -1;
  return (int)launch(sample_kernel, dim3(p->batch), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, *p);
}

int rlz_penalties(float* logits, long long ld, int vocab, int batch, const int32_t* history, int window, const float* repetition,
                  const float* presence, const float* frequency, void* stream) {
  return (int)launch(penalties_kernel, dim3(batch), dim3(256), 0, (cudaStream_t)stream, logits, (int64_t)ld, vocab, history, window,
                     repetition, presence, frequency);
}

int rlz_sizeof_sample_params() { return (int)sizeof(rlz::SampleParams); }
int rlz_sizeof_shard_sample() { return (int)sizeof(rlz::ShardSample); }

// Vocabulary-sharded sampling, first half: p.logits / p.vocab describe this rank's slice; candidates go to every rank's inbox.
int rlz_sample_push(const SampleParams* p, const ShardSample* c, void* stream) {
  if (p->batch < 1 || p->batch > c->batch_cap || c->K < 1 || c->K > SAMP_MAX_CAND || c->world < 1 || c->world > GEMV_AR_MAX_RANKS) return -1;
  return (int)launch(sample_push_kernel, dim3(p->batch), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, *p, *c);
}
// Second half: the draw over the gathered candidates; p.logits is not read.
int rlz_sample_merge(const SampleParams* p, const ShardSample* c, void* stream) {
  if (p->batch < 1 || p->batch > c->batch_cap || c->K < 1 || c->K > SAMP_MAX_CAND || c->world < 1 || c->world > GEMV_AR_MAX_RANKS) return -1;
  return (int)launch(sample_merge_kernel, dim3(p->batch), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, *p, *c);
}

}  // extern "C"
