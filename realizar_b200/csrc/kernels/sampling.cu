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

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(const __grid_constant__ SampleParams p) {
  __shared__ float sval[33]; __shared__ int sidx[33];
  __shared__ unsigned hist[256];
  __shared__ float cval[SAMP_MAX_CAND]; __shared__ int cidx[SAMP_MAX_CAND];
  __shared__ float csum[SAMP_MAX_CAND];
  __shared__ unsigned sh_prefix, sh_kk, sh_count, sh_ties;
  __shared__ int sh_pick;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const float* row = p.logits + (int64_t)b * p.ld;
  const int V = p.vocab;
  const float temp = p.temperature[b];
  int k = p.top_k[b];

  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = tid; i < V; i += SAMP_THREADS) { const float v = row[i]; if (v > best) { best = v; bi = i; } }
  float vmax; int imax;
  block_argmax(best, bi, sval, sidx, &vmax, &imax);
  if (temp <= 0.f || k == 1) { if (tid == 0) { p.out[b] = imax; if (p.out_logprob) p.out_logprob[b] = 0.f; } return; }
  if (k <= 0 || k > SAMP_MAX_CAND) k = SAMP_MAX_CAND;
  if (k > V) k = V;

  // ---- exact k-th largest key by 4 x 8-bit radix select ------------------------------------
  if (tid == 0) { sh_prefix = 0; sh_kk = (unsigned)k; }
  for (int round = 0; round < 4; ++round) {
    const int shift = 24 - 8 * round;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = sh_prefix, pmask = round == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += SAMP_THREADS) {
      const uint32_t key = float_key(row[i]);
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFFu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned cum = 0, kk = sh_kk; int bin = 255;
      for (; bin > 0; --bin) { if (cum + hist[bin] >= kk) break; cum += hist[bin]; }
      sh_kk = kk - cum;                       // still needed from inside this bin
      sh_prefix = prefix | ((unsigned)bin << shift);
    }
    __syncthreads();
  }
  const uint32_t tkey = sh_prefix;            // key of the k-th largest logit
  const unsigned ties_wanted = sh_kk;         // how many elements equal to it belong to the top k
  if (tid == 0) { sh_count = 0; sh_ties = 0; }
  for (int i = tid; i < SAMP_MAX_CAND; i += SAMP_THREADS) { cval[i] = -INFINITY; cidx[i] = 0x7fffffff; }
  __syncthreads();
  for (int i = tid; i < V; i += SAMP_THREADS) {
    const float v = row[i]; const uint32_t key = float_key(v);
    bool take = key > tkey;
    if (key == tkey) take = atomicAdd(&sh_ties, 1u) < ties_wanted;
    if (take) { const unsigned slot = atomicAdd(&sh_count, 1u); if (slot < SAMP_MAX_CAND) { cval[slot] = v; cidx[slot] = i; } }
  }
  __syncthreads();

  // ---- bitonic sort: value descending, index ascending --------------------------------------
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

  // ---- softmax over candidates, min-p / top-p filtering, inverse-CDF draw --------------------
  const int n = (int)min(sh_count, (unsigned)SAMP_MAX_CAND);
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
  if (tid == 0) sh_pick = n - 1;
  __syncthreads();
  // nucleus: smallest prefix whose mass reaches top_p * total
  float kept = total;
  if (top_p < 1.f) {
    const float need = top_p * total;
    const bool here = csum[tid] >= need && (tid == 0 || csum[tid - 1] < need);
    if (here) sh_pick = tid;
    __syncthreads();
    kept = csum[sh_pick];
    __syncthreads();
  }
  const int last = top_p < 1.f ? sh_pick : n - 1;
  const float target = p.uniform[b] * kept;
  if (tid == 0) sh_pick = last;
  __syncthreads();
  if (tid <= last && csum[tid] > target && (tid == 0 || csum[tid - 1] <= target)) sh_pick = tid;
  __syncthreads();
  if (tid == 0) {
    const int c = sh_pick;
    p.out[b] = cidx[c];
    if (p.out_logprob) { const float pc = c == 0 ? csum[0] : csum[c] - csum[c - 1]; p.out_logprob[b] = logf(fmaxf(pc, 1e-30f) / kept); }
  }
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

}  // extern "C"
