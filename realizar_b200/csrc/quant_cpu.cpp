// Host-side quantisation library: ggml-layout quantisers, dequantisers and fused
// dequant-dot matrix-vector products (scalar + AVX2, runtime dispatched), with a small
// persistent thread pool for row-parallel matvec.
//
// Capability parity with the reference's CPU compute layer
// (src/quantize/fused_k.rs, fused_q5k_q6k.rs, parallel_k.rs, activation.rs, encode.rs):
// activations are quantised once per matvec to Q8_K (K-quants) or Q8_0 (legacy blocks)
// and every weight row is consumed in its on-disk block layout.
#include "quant_blocks.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#define RLZ_X86 1
#endif

using namespace rlz;

namespace {

// ------------------------------------------------------------------ thread pool ------
// Workers spin for a few microseconds on the epoch word before they go to sleep on the condition variable: a decoder
// issues a couple of hundred small matrix-vector products per token, and a futex wake per product would cost more than
// the products themselves.
class Pool {
 public:
  explicit Pool(int n) : n_(std::max(1, n)) {
    for (int i = 1; i < n_; ++i) workers_.emplace_back([this, i] { loop(i); });
  }
  ~Pool() {
    { std::lock_guard<std::mutex> l(mu_); stop_ = true; epoch_.fetch_add(1, std::memory_order_release); }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  int size() const { return n_; }
  // run fn(worker_index) on every worker (including the caller as worker 0)
  void run(const std::function<void(int)>& fn) {
    if (n_ == 1) { fn(0); return; }
    std::lock_guard<std::mutex> one_caller(run_mu_);      // callers on different threads take turns (the hand-over state is single)
    {
      std::lock_guard<std::mutex> l(mu_);
      fn_ = &fn;
      pending_.store(n_ - 1, std::memory_order_relaxed);
      epoch_.fetch_add(1, std::memory_order_release);
    }
    if (sleepers_.load(std::memory_order_acquire) > 0) cv_.notify_all();
    fn(0);
    for (int spins = 0; pending_.load(std::memory_order_acquire) != 0; ++spins) {
      if (spins < 20000) cpu_relax(); else std::this_thread::yield();
    }
    fn_ = nullptr;
  }
 private:
  static void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#endif
  }
  void loop(int idx) {
    uint64_t seen = 0;
    for (;;) {
      int spins = 0;
      while (epoch_.load(std::memory_order_acquire) == seen) {
        if (++spins < 4000) { cpu_relax(); continue; }
        std::unique_lock<std::mutex> l(mu_);
        sleepers_.fetch_add(1, std::memory_order_release);
        cv_.wait(l, [&] { return epoch_.load(std::memory_order_acquire) != seen; });
        sleepers_.fetch_sub(1, std::memory_order_release);
      }
      seen = epoch_.load(std::memory_order_acquire);
      if (stop_) return;
      const std::function<void(int)>* fn = fn_;
      if (fn) (*fn)(idx);
      pending_.fetch_sub(1, std::memory_order_release);
    }
  }
  int n_;
  std::vector<std::thread> workers_;
  std::mutex mu_, run_mu_;
  std::condition_variable cv_;
  const std::function<void(int)>* fn_ = nullptr;
  std::atomic<int> pending_{0}, sleepers_{0};
  std::atomic<uint64_t> epoch_{0};
  bool stop_ = false;
};

Pool* g_pool = nullptr;
std::mutex g_pool_mu;

Pool& pool() {
  std::lock_guard<std::mutex> l(g_pool_mu);
  if (!g_pool) {
    int n = (int)std::thread::hardware_concurrency();
    if (const char* e = std::getenv("RLZ_CPU_THREADS")) n = std::atoi(e);
    g_pool = new Pool(std::max(1, std::min(n, 64)));
  }
  return *g_pool;
}

inline int nearest_int(float f) { return (int)lrintf(f); }

// ------------------------------------------------------------------ quantisers -------
void quantize_row_q4_0(const float* x, uint8_t* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float amax = 0.f, mx = 0.f;
    for (int j = 0; j < 32; ++j) { float v = x[i * 32 + j]; if (fabsf(v) > amax) { amax = fabsf(v); mx = v; } }
    const float d = mx / -8.f; const float id = d ? 1.f / d : 0.f;
    uint8_t* b = y + i * 18; uint16_t h = float_to_half_bits(d); b[0] = h & 0xFF; b[1] = h >> 8;
    for (int j = 0; j < 16; ++j) {
      const uint8_t a = (uint8_t)std::min(15, (int)(x[i * 32 + j] * id + 8.5f));
      const uint8_t c = (uint8_t)std::min(15, (int)(x[i * 32 + 16 + j] * id + 8.5f));
      b[2 + j] = a | (c << 4);
    }
  }
}
void quantize_row_q4_1(const float* x, uint8_t* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float mn = x[i * 32], mx = x[i * 32];
    for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[i * 32 + j]); mx = std::max(mx, x[i * 32 + j]); }
    const float d = (mx - mn) / 15.f, id = d ? 1.f / d : 0.f;
    uint8_t* b = y + i * 20; uint16_t h = float_to_half_bits(d), hm = float_to_half_bits(mn);
    b[0] = h & 0xFF; b[1] = h >> 8; b[2] = hm & 0xFF; b[3] = hm >> 8;
    for (int j = 0; j < 16; ++j) {
      const uint8_t a = (uint8_t)std::min(15, (int)((x[i * 32 + j] - mn) * id + 0.5f));
      const uint8_t c = (uint8_t)std::min(15, (int)((x[i * 32 + 16 + j] - mn) * id + 0.5f));
      b[4 + j] = a | (c << 4);
    }
  }
}
void quantize_row_q5_0(const float* x, uint8_t* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float amax = 0.f, mx = 0.f;
    for (int j = 0; j < 32; ++j) { float v = x[i * 32 + j]; if (fabsf(v) > amax) { amax = fabsf(v); mx = v; } }
    const float d = mx / -16.f, id = d ? 1.f / d : 0.f;
    uint8_t* b = y + i * 22; uint16_t h = float_to_half_bits(d); b[0] = h & 0xFF; b[1] = h >> 8;
    uint32_t qh = 0;
    for (int j = 0; j < 16; ++j) {
      const uint8_t a = (uint8_t)std::min(31, (int)(x[i * 32 + j] * id + 16.5f));
      const uint8_t c = (uint8_t)std::min(31, (int)(x[i * 32 + 16 + j] * id + 16.5f));
      b[6 + j] = (a & 0xF) | ((c & 0xF) << 4);
      qh |= (uint32_t)((a & 0x10) >> 4) << j;
      qh |= (uint32_t)((c & 0x10) >> 4) << (j + 16);
    }
    memcpy(b + 2, &qh, 4);
  }
}
void quantize_row_q5_1(const float* x, uint8_t* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float mn = x[i * 32], mx = x[i * 32];
    for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[i * 32 + j]); mx = std::max(mx, x[i * 32 + j]); }
    const float d = (mx - mn) / 31.f, id = d ? 1.f / d : 0.f;
    uint8_t* b = y + i * 24; uint16_t h = float_to_half_bits(d), hm = float_to_half_bits(mn);
    b[0] = h & 0xFF; b[1] = h >> 8; b[2] = hm & 0xFF; b[3] = hm >> 8;
    uint32_t qh = 0;
    for (int j = 0; j < 16; ++j) {
      const uint8_t a = (uint8_t)std::min(31, (int)((x[i * 32 + j] - mn) * id + 0.5f));
      const uint8_t c = (uint8_t)std::min(31, (int)((x[i * 32 + 16 + j] - mn) * id + 0.5f));
      b[8 + j] = (a & 0xF) | ((c & 0xF) << 4);
      qh |= (uint32_t)((a & 0x10) >> 4) << j;
      qh |= (uint32_t)((c & 0x10) >> 4) << (j + 16);
    }
    memcpy(b + 4, &qh, 4);
  }
}
void quantize_row_q8_0(const float* x, uint8_t* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[i * 32 + j]));
    const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
    uint8_t* b = y + i * 34; uint16_t h = float_to_half_bits(d); b[0] = h & 0xFF; b[1] = h >> 8;
    for (int j = 0; j < 32; ++j) ((int8_t*)(b + 2))[j] = (int8_t)nearest_int(x[i * 32 + j] * id);
  }
}

// Weighted affine fit x ~ scale*L - min over L in [0, nmax] for one sub-block
// (iterated grid search over candidate inverse scales, least-squares refit of scale/min).
float fit_scale_min(int n, int nmax, const float* x, const float* w, uint8_t* L, float* the_min,
                    uint8_t* Laux, float rmin, float rdelta, int nstep) {
  float mn = x[0], mx = x[0], sum_w = w[0], sum_x = w[0] * x[0];
  for (int i = 1; i < n; ++i) {
    mn = std::min(mn, x[i]); mx = std::max(mx, x[i]);
    sum_w += w[i]; sum_x += w[i] * x[i];
  }
  if (mn > 0) mn = 0;
  if (mx == mn) { for (int i = 0; i < n; ++i) L[i] = 0; *the_min = -mn; return 0.f; }
  float iscale = nmax / (mx - mn), scale = 1.f / iscale, best = 0.f;
  for (int i = 0; i < n; ++i) {
    int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - mn))));
    L[i] = (uint8_t)l;
    float diff = scale * l + mn - x[i];
    best += w[i] * diff * diff;
  }
  for (int is = 0; is <= nstep; ++is) {
    iscale = (rmin + rdelta * is + nmax) / (mx - mn);
    float sum_l = 0, sum_l2 = 0, sum_xl = 0;
    for (int i = 0; i < n; ++i) {
      int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - mn))));
      Laux[i] = (uint8_t)l;
      sum_l += w[i] * l; sum_l2 += w[i] * l * l; sum_xl += w[i] * l * x[i];
    }
    float D = sum_w * sum_l2 - sum_l * sum_l;
    if (D > 0) {
      float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
      float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
      if (this_min > 0) { this_min = 0; this_scale = sum_l2 > 0 ? sum_xl / sum_l2 : 0.f; }
      float err = 0;
      for (int i = 0; i < n; ++i) { float diff = this_scale * Laux[i] + this_min - x[i]; err += w[i] * diff * diff; }
      if (err < best) { memcpy(L, Laux, n); best = err; scale = this_scale; mn = this_min; }
    }
  }
  *the_min = -mn;
  return scale;
}

void pack_k4_scales(const float* scales, const float* mins, uint8_t* packed, float* d_out, float* dmin_out) {
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; ++j) { max_scale = std::max(max_scale, scales[j]); max_min = std::max(max_min, mins[j]); }
  const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
  const float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
  memset(packed, 0, 12);
  for (int j = 0; j < 8; ++j) {
    uint8_t ls = (uint8_t)std::min(63, nearest_int(inv_scale * scales[j]));
    uint8_t lm = (uint8_t)std::min(63, nearest_int(inv_min * mins[j]));
    if (j < 4) { packed[j] = ls; packed[j + 4] = lm; }
    else {
      packed[j + 4] = (ls & 0xF) | ((lm & 0xF) << 4);
      packed[j - 4] |= (uint8_t)((ls >> 4) << 6);
      packed[j] |= (uint8_t)((lm >> 4) << 6);
    }
  }
  *d_out = max_scale / 63.f; *dmin_out = max_min / 63.f;
}

void quantize_row_q4_k(const float* x, uint8_t* y, int64_t k) {
  uint8_t L[256], Laux[32]; float weights[32], mins[8], scales[8];
  for (int64_t i = 0; i < k / 256; ++i, x += 256, y += 144) {
    for (int j = 0; j < 8; ++j) {
      float sum_x2 = 0; for (int l = 0; l < 32; ++l) sum_x2 += x[32 * j + l] * x[32 * j + l];
      float av_x = sqrtf(sum_x2 / 32);
      for (int l = 0; l < 32; ++l) weights[l] = av_x + fabsf(x[32 * j + l]);
      scales[j] = fit_scale_min(32, 15, x + 32 * j, weights, L + 32 * j, &mins[j], Laux, -1.f, 0.1f, 20);
    }
    float d, dmin; pack_k4_scales(scales, mins, y + 4, &d, &dmin);
    uint16_t hd = float_to_half_bits(d), hm = float_to_half_bits(dmin);
    y[0] = hd & 0xFF; y[1] = hd >> 8; y[2] = hm & 0xFF; y[3] = hm >> 8;
    const float fd = half_bits_to_float(hd), fm = half_bits_to_float(hm);
    for (int j = 0; j < 8; ++j) {
      uint8_t sc, m; get_scale_min_k4(j, y + 4, &sc, &m);
      const float d1 = fd * sc; if (!d1) { for (int l = 0; l < 32; ++l) L[32 * j + l] = 0; continue; }
      const float dm = fm * m;
      for (int l = 0; l < 32; ++l) L[32 * j + l] = (uint8_t)std::max(0, std::min(15, nearest_int((x[32 * j + l] + dm) / d1)));
    }
    uint8_t* q = y + 16;
    for (int j = 0; j < 256; j += 64) { for (int l = 0; l < 32; ++l) q[l] = L[j + l] | (L[j + l + 32] << 4); q += 32; }
  }
}

void quantize_row_q5_k(const float* x, uint8_t* y, int64_t k) {
  uint8_t L[256], Laux[32]; float weights[32], mins[8], scales[8];
  for (int64_t i = 0; i < k / 256; ++i, x += 256, y += 176) {
    for (int j = 0; j < 8; ++j) {
      float sum_x2 = 0; for (int l = 0; l < 32; ++l) sum_x2 += x[32 * j + l] * x[32 * j + l];
      float av_x = sqrtf(sum_x2 / 32);
      for (int l = 0; l < 32; ++l) weights[l] = av_x + fabsf(x[32 * j + l]);
      scales[j] = fit_scale_min(32, 31, x + 32 * j, weights, L + 32 * j, &mins[j], Laux, -0.5f, 0.1f, 15);
    }
    float d, dmin; pack_k4_scales(scales, mins, y + 4, &d, &dmin);
    uint16_t hd = float_to_half_bits(d), hm = float_to_half_bits(dmin);
    y[0] = hd & 0xFF; y[1] = hd >> 8; y[2] = hm & 0xFF; y[3] = hm >> 8;
    const float fd = half_bits_to_float(hd), fm = half_bits_to_float(hm);
    for (int j = 0; j < 8; ++j) {
      uint8_t sc, m; get_scale_min_k4(j, y + 4, &sc, &m);
      const float d1 = fd * sc; if (!d1) { for (int l = 0; l < 32; ++l) L[32 * j + l] = 0; continue; }
      const float dm = fm * m;
      for (int l = 0; l < 32; ++l) L[32 * j + l] = (uint8_t)std::max(0, std::min(31, nearest_int((x[32 * j + l] + dm) / d1)));
    }
    uint8_t* qh = y + 16; uint8_t* ql = y + 48; memset(qh, 0, 32);
    uint8_t m1 = 1, m2 = 2;
    for (int n = 0; n < 256; n += 64) {
      for (int j = 0; j < 32; ++j) {
        int l1 = L[n + j]; if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
        int l2 = L[n + j + 32]; if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
        ql[j] = (uint8_t)(l1 | (l2 << 4));
      }
      m1 = (uint8_t)(m1 << 2); m2 = (uint8_t)(m2 << 2); ql += 32;
    }
  }
}

// symmetric fit x ~ scale*L, L in [-nmax, nmax-1]; returns scale, writes L+nmax
float fit_scale_sym(int n, int nmax, const float* x, int8_t* L) {
  float amax = 0, mx = 0;
  for (int i = 0; i < n; ++i) { float ax = fabsf(x[i]); if (ax > amax) { amax = ax; mx = x[i]; } }
  if (amax < 1e-30f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.f; }
  float best_scale = 0, best_err = -1;
  for (int is = -9; is <= 9; ++is) {
    float iscale = -(nmax + 0.1f * is) / mx;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
      int l = std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
      float w = x[i] * x[i];
      sumlx += w * x[i] * l; suml2 += w * l * l;
    }
    if (suml2 <= 0) continue;
    float scale = sumlx / suml2, err = 0;
    for (int i = 0; i < n; ++i) {
      int l = std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
      float diff = scale * l - x[i]; err += x[i] * x[i] * diff * diff;
    }
    if (best_err < 0 || err < best_err) { best_err = err; best_scale = scale; }
  }
  float iscale = best_scale ? 1.f / best_scale : 0.f;
  for (int i = 0; i < n; ++i) L[i] = (int8_t)std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
  return best_scale;
}

void quantize_row_q6_k(const float* x, uint8_t* y, int64_t k) {
  int8_t L[256]; float scales[16];
  for (int64_t i = 0; i < k / 256; ++i, x += 256, y += 210) {
    float max_scale = 0, max_abs_scale = 0;
    for (int ib = 0; ib < 16; ++ib) {
      float s = fit_scale_sym(16, 32, x + 16 * ib, L + 16 * ib);
      scales[ib] = s;
      if (fabsf(s) > max_abs_scale) { max_abs_scale = fabsf(s); max_scale = s; }
    }
    if (max_abs_scale < 1e-30f) { memset(y, 0, 210); continue; }
    const float iscale = -128.f / max_scale;
    uint16_t hd = float_to_half_bits(1.f / iscale);
    y[208] = hd & 0xFF; y[209] = hd >> 8;
    int8_t* sc = (int8_t*)(y + 192);
    for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
    const float fd = half_bits_to_float(hd);
    uint8_t Lu[256];
    for (int j = 0; j < 16; ++j) {
      const float d = fd * sc[j];
      for (int ii = 0; ii < 16; ++ii) {
        int l = d ? nearest_int(x[16 * j + ii] / d) : 0;
        Lu[16 * j + ii] = (uint8_t)(std::max(-32, std::min(31, l)) + 32);
      }
    }
    uint8_t* ql = y; uint8_t* qh = y + 128;
    for (int j = 0; j < 256; j += 128) {
      for (int l = 0; l < 32; ++l) {
        const uint8_t q1 = Lu[j + l] & 0xF, q2 = Lu[j + l + 32] & 0xF, q3 = Lu[j + l + 64] & 0xF, q4 = Lu[j + l + 96] & 0xF;
        ql[l] = q1 | (q3 << 4); ql[l + 32] = q2 | (q4 << 4);
        qh[l] = (uint8_t)((Lu[j + l] >> 4) | ((Lu[j + l + 32] >> 4) << 2) | ((Lu[j + l + 64] >> 4) << 4) | ((Lu[j + l + 96] >> 4) << 6));
      }
      ql += 64; qh += 32;
    }
  }
}

void quantize_row_q2_k(const float* x, uint8_t* y, int64_t k) {
  uint8_t L[256], Laux[16]; float weights[16], mins[16], scales[16];
  for (int64_t i = 0; i < k / 256; ++i, x += 256, y += 84) {
    float max_scale = 0, max_min = 0;
    for (int j = 0; j < 16; ++j) {
      for (int l = 0; l < 16; ++l) weights[l] = fabsf(x[16 * j + l]);
      scales[j] = fit_scale_min(16, 3, x + 16 * j, weights, L + 16 * j, &mins[j], Laux, -0.5f, 0.1f, 15);
      max_scale = std::max(max_scale, scales[j]); max_min = std::max(max_min, mins[j]);
    }
    uint8_t* sc = y; float d = 0, dmin = 0;
    if (max_scale > 0) { float iscale = 15.f / max_scale; for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)nearest_int(iscale * scales[j]); d = max_scale / 15.f; }
    else memset(sc, 0, 16);
    if (max_min > 0) { float iscale = 15.f / max_min; for (int j = 0; j < 16; ++j) sc[j] |= (uint8_t)(nearest_int(iscale * mins[j]) << 4); dmin = max_min / 15.f; }
    uint16_t hd = float_to_half_bits(d), hm = float_to_half_bits(dmin);
    y[80] = hd & 0xFF; y[81] = hd >> 8; y[82] = hm & 0xFF; y[83] = hm >> 8;
    const float fd = half_bits_to_float(hd), fm = half_bits_to_float(hm);
    for (int j = 0; j < 16; ++j) {
      const float dd = fd * (sc[j] & 0xF); const float dm = fm * (sc[j] >> 4);
      for (int ii = 0; ii < 16; ++ii)
        L[16 * j + ii] = dd ? (uint8_t)std::max(0, std::min(3, nearest_int((x[16 * j + ii] + dm) / dd))) : 0;
    }
    uint8_t* q = y + 16;
    for (int j = 0; j < 256; j += 128)
      for (int l = 0; l < 32; ++l)
        q[j / 4 + l] = L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6);
  }
}

// ------------------------------------------------------------------ activations ------
struct Q8K { float d; int8_t qs[256]; int16_t bsums[16]; };

void quantize_q8_k(const float* x, Q8K* y, int64_t k) {
  for (int64_t i = 0; i < k / 256; ++i, x += 256) {
    float amax = 0, mx = 0;
    for (int j = 0; j < 256; ++j) { float ax = fabsf(x[j]); if (ax > amax) { amax = ax; mx = x[j]; } }
    if (!amax) { y[i].d = 0; memset(y[i].qs, 0, 256); memset(y[i].bsums, 0, 32); continue; }
    const float iscale = -127.f / mx;
    for (int j = 0; j < 256; ++j) y[i].qs[j] = (int8_t)std::min(127, nearest_int(iscale * x[j]));
    for (int j = 0; j < 16; ++j) { int s = 0; for (int l = 0; l < 16; ++l) s += y[i].qs[16 * j + l]; y[i].bsums[j] = (int16_t)s; }
    y[i].d = 1.f / iscale;
  }
}

struct Q80A { float d; int32_t sum; int8_t qs[32]; };     // sum of the 32 codes: the offset term of the unsigned weight types
void quantize_q8_0_act(const float* x, Q80A* y, int64_t k) {
  for (int64_t i = 0; i < k / 32; ++i) {
    float amax = 0; for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[i * 32 + j]));
    const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
    int sum = 0;
    y[i].d = d; for (int j = 0; j < 32; ++j) { y[i].qs[j] = (int8_t)nearest_int(x[i * 32 + j] * id); sum += y[i].qs[j]; }
    y[i].sum = sum;
  }
}

// ------------------------------------------------------------------ fused dots -------
float dot_q4k_q8k_scalar(const uint8_t* w, const Q8K* a, int nb) {
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 144) {
    const float d = half_bits_to_float(load_u16(w)) * a[i].d, dmin = half_bits_to_float(load_u16(w + 2)) * a[i].d;
    const uint8_t* q = w + 16; const int8_t* q8 = a[i].qs;
    int sumi = 0, summ = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      int lo = 0, hi = 0;
      for (int l = 0; l < 32; ++l) { lo += (q[l] & 0xF) * q8[l]; hi += (q[l] >> 4) * q8[32 + l]; }
      sumi += sc0 * lo + sc1 * hi;
      summ += m0 * (a[i].bsums[4 * j] + a[i].bsums[4 * j + 1]) + m1 * (a[i].bsums[4 * j + 2] + a[i].bsums[4 * j + 3]);
      q += 32; q8 += 64;
    }
    sumf += d * sumi - dmin * summ;
  }
  return sumf;
}
float dot_q5k_q8k_scalar(const uint8_t* w, const Q8K* a, int nb) {
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 176) {
    const float d = half_bits_to_float(load_u16(w)) * a[i].d, dmin = half_bits_to_float(load_u16(w + 2)) * a[i].d;
    const uint8_t* qh = w + 16; const uint8_t* q = w + 48; const int8_t* q8 = a[i].qs;
    int sumi = 0, summ = 0; uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      int lo = 0, hi = 0;
      for (int l = 0; l < 32; ++l) {
        lo += ((q[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) * q8[l];
        hi += ((q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) * q8[32 + l];
      }
      sumi += sc0 * lo + sc1 * hi;
      summ += m0 * (a[i].bsums[4 * j] + a[i].bsums[4 * j + 1]) + m1 * (a[i].bsums[4 * j + 2] + a[i].bsums[4 * j + 3]);
      q += 32; q8 += 64; u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
    }
    sumf += d * sumi - dmin * summ;
  }
  return sumf;
}
float dot_q6k_q8k_scalar(const uint8_t* w, const Q8K* a, int nb) {
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 210) {
    const uint8_t* ql = w; const uint8_t* qh = w + 128; const int8_t* sc = (const int8_t*)(w + 192);
    const float d = half_bits_to_float(load_u16(w + 208)) * a[i].d; const int8_t* q8 = a[i].qs;
    int sumi = 0;
    for (int n = 0; n < 2; ++n) {
      int s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int l = 0; l < 32; ++l) {
        const int is = l / 16;
        s[is + 0] += ((int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32) * q8[l];
        s[is + 2] += ((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32) * q8[l + 32];
        s[is + 4] += ((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32) * q8[l + 64];
        s[is + 6] += ((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32) * q8[l + 96];
      }
      for (int t = 0; t < 8; ++t) sumi += sc[t] * s[t];
      ql += 64; qh += 32; sc += 8; q8 += 128;
    }
    sumf += d * sumi;
  }
  return sumf;
}

#if RLZ_X86
__attribute__((target("avx2,fma"))) inline float hsum8(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi); lo = _mm_hadd_ps(lo, lo); lo = _mm_hadd_ps(lo, lo);
  return _mm_cvtss_f32(lo);
}
__attribute__((target("avx2,fma"))) inline int hsum8i(__m256i v) {
  __m128i lo = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
  lo = _mm_hadd_epi32(lo, lo); lo = _mm_hadd_epi32(lo, lo);
  return _mm_cvtsi128_si32(lo);
}
__attribute__((target("avx2,fma")))
float dot_q4k_q8k_avx2(const uint8_t* w, const Q8K* a, int nb) {
  const __m256i m4 = _mm256_set1_epi8(0xF);
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 144) {
    const float d = half_bits_to_float(load_u16(w)) * a[i].d, dmin = half_bits_to_float(load_u16(w + 2)) * a[i].d;
    const uint8_t* q = w + 16; const int8_t* q8 = a[i].qs;
    __m256i acc = _mm256_setzero_si256(); int summ = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      const __m256i qb = _mm256_loadu_si256((const __m256i*)q);
      const __m256i lo = _mm256_and_si256(qb, m4), hi = _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4);
      const __m256i a0 = _mm256_loadu_si256((const __m256i*)q8), a1 = _mm256_loadu_si256((const __m256i*)(q8 + 32));
      __m256i p0 = _mm256_maddubs_epi16(lo, a0), p1 = _mm256_maddubs_epi16(hi, a1);
      p0 = _mm256_madd_epi16(p0, _mm256_set1_epi16(sc0)); p1 = _mm256_madd_epi16(p1, _mm256_set1_epi16(sc1));
      acc = _mm256_add_epi32(acc, _mm256_add_epi32(p0, p1));
      summ += m0 * (a[i].bsums[4 * j] + a[i].bsums[4 * j + 1]) + m1 * (a[i].bsums[4 * j + 2] + a[i].bsums[4 * j + 3]);
      q += 32; q8 += 64;
    }
    sumf += d * hsum8i(acc) - dmin * summ;
  }
  return sumf;
}
__attribute__((target("avx2,fma")))
float dot_q6k_q8k_avx2(const uint8_t* w, const Q8K* a, int nb) {
  const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), off = _mm256_set1_epi8(32);
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 210) {
    const uint8_t* ql = w; const uint8_t* qh = w + 128; const int8_t* sc = (const int8_t*)(w + 192);
    const float d = half_bits_to_float(load_u16(w + 208)) * a[i].d; const int8_t* q8 = a[i].qs;
    __m256i acc = _mm256_setzero_si256();
    for (int n = 0; n < 2; ++n) {
      const __m256i l0 = _mm256_loadu_si256((const __m256i*)ql), l1 = _mm256_loadu_si256((const __m256i*)(ql + 32));
      const __m256i h = _mm256_loadu_si256((const __m256i*)qh);
      __m256i q[4];
      q[0] = _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_slli_epi16(_mm256_and_si256(h, m2), 4));
      q[1] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4));
      q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4));
      q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4));
      for (int t = 0; t < 4; ++t) {
        const __m256i av = _mm256_loadu_si256((const __m256i*)(q8 + 32 * t));
        // (q-32)*a = q*a - 32*a, both through maddubs with unsigned first operand
        __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(q[t], av), _mm256_maddubs_epi16(off, av));
        // per-16 scales: first 16 lanes (8 x i16) use sc[2t], last 16 use sc[2t+1]
        const __m256i s = _mm256_set_m128i(_mm_set1_epi16(sc[2 * t + 1]), _mm_set1_epi16(sc[2 * t]));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p, s));
      }
      ql += 64; qh += 32; sc += 8; q8 += 128;
    }
    sumf += d * hsum8i(acc);
  }
  return sumf;
}
// Q5_K: as Q4_K with the fifth bit of every weight taken from qh (bit 2j of byte l for sub-block 2j, bit 2j+1 for 2j+1)
__attribute__((target("avx2,fma")))
float dot_q5k_q8k_avx2(const uint8_t* w, const Q8K* a, int nb) {
  const __m256i m4 = _mm256_set1_epi8(0xF), one = _mm256_set1_epi8(1);
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 176) {
    const float d = half_bits_to_float(load_u16(w)) * a[i].d, dmin = half_bits_to_float(load_u16(w + 2)) * a[i].d;
    const __m256i hb = _mm256_loadu_si256((const __m256i*)(w + 16));
    const uint8_t* q = w + 48; const int8_t* q8 = a[i].qs;
    __m256i acc = _mm256_setzero_si256(); int summ = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      const __m256i qb = _mm256_loadu_si256((const __m256i*)q);
      const __m256i h0 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 2 * j), one), 4);
      const __m256i h1 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 2 * j + 1), one), 4);
      const __m256i lo = _mm256_or_si256(_mm256_and_si256(qb, m4), h0), hi = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(qb, 4), m4), h1);
      const __m256i a0 = _mm256_loadu_si256((const __m256i*)q8), a1 = _mm256_loadu_si256((const __m256i*)(q8 + 32));
      __m256i p0 = _mm256_maddubs_epi16(lo, a0), p1 = _mm256_maddubs_epi16(hi, a1);
      p0 = _mm256_madd_epi16(p0, _mm256_set1_epi16(sc0)); p1 = _mm256_madd_epi16(p1, _mm256_set1_epi16(sc1));
      acc = _mm256_add_epi32(acc, _mm256_add_epi32(p0, p1));
      summ += m0 * (a[i].bsums[4 * j] + a[i].bsums[4 * j + 1]) + m1 * (a[i].bsums[4 * j + 2] + a[i].bsums[4 * j + 3]);
      q += 32; q8 += 64;
    }
    sumf += d * hsum8i(acc) - dmin * summ;
  }
  return sumf;
}

// ---- 32-wide blocks (Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q8_0) against Q8_0-quantised activations -----------------------------
// 16 bytes of nibbles -> 32 bytes: low nibbles (elements 0..15) then high nibbles (16..31)
__attribute__((target("avx2"))) inline __m256i nibbles32(const uint8_t* qs) {
  const __m128i q = _mm_loadu_si128((const __m128i*)qs);
  return _mm256_and_si256(_mm256_set_m128i(_mm_srli_epi16(q, 4), q), _mm256_set1_epi8(0xF));
}
// 32 bits -> 32 bytes, 0x10 where the bit is set (the fifth bit of the 5-bit types)
__attribute__((target("avx2"))) inline __m256i fifth_bits(uint32_t x) {
  const __m256i shuf = _mm256_set_epi64x(0x0303030303030303LL, 0x0202020202020202LL, 0x0101010101010101LL, 0x0000000000000000LL);
  const __m256i sel = _mm256_set1_epi64x((long long)0x8040201008040201ULL);
  const __m256i b = _mm256_and_si256(_mm256_shuffle_epi8(_mm256_set1_epi32((int)x), shuf), sel);
  return _mm256_and_si256(_mm256_cmpeq_epi8(b, sel), _mm256_set1_epi8(0x10));
}
__attribute__((target("avx2,fma")))
float dot_legacy_q8_0_avx2(int qtype, const uint8_t* w, const Q80A* a, int nb) {
  const __m256i ones16 = _mm256_set1_epi16(1);
  __m256 acc = _mm256_setzero_ps();
  float extra = 0.f;                                       // minimum terms of Q4_1 / Q5_1
  const int bb = qtype_block_bytes(qtype);
  for (int i = 0; i < nb; ++i, w += bb) {
    const __m256i av = _mm256_loadu_si256((const __m256i*)a[i].qs);
    const float d = half_bits_to_float(load_u16(w));
    __m256i p;
    switch (qtype) {
      case QT_Q8_0: {
        const __m256i q = _mm256_loadu_si256((const __m256i*)(w + 2));
        p = _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_sign_epi8(q, q), _mm256_sign_epi8(av, q)), ones16);
        break; }
      case QT_Q4_0: {
        const __m256i q = nibbles32(w + 2);
        p = _mm256_madd_epi16(_mm256_sub_epi16(_mm256_maddubs_epi16(q, av), _mm256_maddubs_epi16(_mm256_set1_epi8(8), av)), ones16);
        break; }
      case QT_Q5_0: {
        const __m256i q = _mm256_or_si256(nibbles32(w + 6), fifth_bits((uint32_t)w[2] | ((uint32_t)w[3] << 8) | ((uint32_t)w[4] << 16) | ((uint32_t)w[5] << 24)));
        p = _mm256_madd_epi16(_mm256_sub_epi16(_mm256_maddubs_epi16(q, av), _mm256_maddubs_epi16(_mm256_set1_epi8(16), av)), ones16);
        break; }
      case QT_Q4_1: case QT_Q5_1: {
        const float m = half_bits_to_float(load_u16(w + 2));
        const __m256i q = qtype == QT_Q4_1 ? nibbles32(w + 4)
            : _mm256_or_si256(nibbles32(w + 8), fifth_bits((uint32_t)w[4] | ((uint32_t)w[5] << 8) | ((uint32_t)w[6] << 16) | ((uint32_t)w[7] << 24)));
        p = _mm256_madd_epi16(_mm256_maddubs_epi16(q, av), ones16);
        extra += m * a[i].d * (float)hsum8i(_mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_set1_epi8(1), av), ones16));
        break; }
      default: return 0.f;
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d * a[i].d), _mm256_cvtepi32_ps(p), acc);
  }
  return hsum8(acc) + extra;
}

// 32-weight block types with VNNI (256-bit form): one dpbusd per block replaces the maddubs / madd pair, the fifth bits of
// Q5_0 / Q5_1 come from a byte mask register loaded with the 32 bits themselves, and the constant offset of the unsigned codes
// (8 for Q4_0, 16 for Q5_0) is applied through the activation block's code sum instead of a second product.
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni,avx2,fma")))
float dot_legacy_q8_0_vnni(int qtype, const uint8_t* w, const Q80A* a, int nb) {
  const __m256i bit5 = _mm256_set1_epi8(0x10);
  __m256 acc = _mm256_setzero_ps();
  float extra = 0.f;
  const int bb = qtype_block_bytes(qtype);
  for (int i = 0; i < nb; ++i, w += bb) {
    const __m256i av = _mm256_loadu_si256((const __m256i*)a[i].qs);
    const float da = half_bits_to_float(load_u16(w)) * a[i].d;
    __m256i p;
    switch (qtype) {
      case QT_Q8_0: {
        const __m256i q = _mm256_loadu_si256((const __m256i*)(w + 2));
        p = _mm256_dpbusd_epi32(_mm256_setzero_si256(), _mm256_sign_epi8(q, q), _mm256_sign_epi8(av, q));
        break; }
      case QT_Q4_0:
        p = _mm256_dpbusd_epi32(_mm256_setzero_si256(), nibbles32(w + 2), av);
        extra = fmaf(-8.f * da, (float)a[i].sum, extra);
        break;
      case QT_Q5_0: {
        const __mmask32 k5 = (__mmask32)((uint32_t)w[2] | ((uint32_t)w[3] << 8) | ((uint32_t)w[4] << 16) | ((uint32_t)w[5] << 24));
        p = _mm256_dpbusd_epi32(_mm256_setzero_si256(), _mm256_or_si256(nibbles32(w + 6), _mm256_maskz_mov_epi8(k5, bit5)), av);
        extra = fmaf(-16.f * da, (float)a[i].sum, extra);
        break; }
      case QT_Q4_1: case QT_Q5_1: {
        const float m = half_bits_to_float(load_u16(w + 2));
        __m256i q;
        if (qtype == QT_Q4_1) q = nibbles32(w + 4);
        else {
          const __mmask32 k5 = (__mmask32)((uint32_t)w[4] | ((uint32_t)w[5] << 8) | ((uint32_t)w[6] << 16) | ((uint32_t)w[7] << 24));
          q = _mm256_or_si256(nibbles32(w + 8), _mm256_maskz_mov_epi8(k5, bit5));
        }
        p = _mm256_dpbusd_epi32(_mm256_setzero_si256(), q, av);
        extra = fmaf(m * a[i].d, (float)a[i].sum, extra);
        break; }
      default: return 0.f;
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(da), _mm256_cvtepi32_ps(p), acc);
  }
  return hsum8(acc) + extra;
}

// ---- AVX-512 VNNI: one dpbusd does the byte products and their 4-wise sums ----------------------------------------------
// Q4_K: the 64 activation bytes of a group of two sub-blocks are contiguous, so one 512-bit operand holds the low nibbles
// (sub-block 2j) in its lower half and the high nibbles (2j + 1) in its upper half; the two sub-block scales sit in the
// matching halves of a multiplier vector.
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni")))
float dot_q4k_q8k_vnni(const uint8_t* w, const Q8K* a, int nb) {
  const __m256i m4 = _mm256_set1_epi8(0xF);
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 144) {
    const float d = half_bits_to_float(load_u16(w)) * a[i].d, dmin = half_bits_to_float(load_u16(w + 2)) * a[i].d;
    const uint8_t* q = w + 16; const int8_t* q8 = a[i].qs;
    __m512i acc = _mm512_setzero_si512(); int summ = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      const __m256i qb = _mm256_loadu_si256((const __m256i*)q);
      const __m512i wv = _mm512_inserti64x4(_mm512_castsi256_si512(_mm256_and_si256(qb, m4)), _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4), 1);
      const __m512i p = _mm512_dpbusd_epi32(_mm512_setzero_si512(), wv, _mm512_loadu_si512((const void*)q8));
      const __m512i scv = _mm512_inserti64x4(_mm512_castsi256_si512(_mm256_set1_epi32(sc0)), _mm256_set1_epi32(sc1), 1);
      acc = _mm512_add_epi32(acc, _mm512_mullo_epi32(p, scv));
      summ += m0 * (a[i].bsums[4 * j] + a[i].bsums[4 * j + 1]) + m1 * (a[i].bsums[4 * j + 2] + a[i].bsums[4 * j + 3]);
      q += 32; q8 += 64;
    }
    sumf = fmaf(-dmin, (float)summ, fmaf(d, (float)_mm512_reduce_add_epi32(acc), sumf));      // (explicit: the x4 form must round alike)
  }
  return sumf;
}
// The same dot for FOUR activation rows against one weight row: the weight's nibbles are unpacked and its sub-block scales
// broadcast once, then multiplied with each activation (prompt chunks: every weight row meets many activation rows).  Per row
// the integer sums and the order of the float operations equal dot_q4k_q8k_vnni, so the results are bit-identical to it.
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni")))
void dot_q4k_q8k_vnni_x4(const uint8_t* w, const Q8K* a, int64_t a_stride, int nb, float* out) {
  const __m256i m4 = _mm256_set1_epi8(0xF);
  float sumf[4] = {0, 0, 0, 0};
  for (int i = 0; i < nb; ++i, w += 144) {
    const float dw = half_bits_to_float(load_u16(w)), dminw = half_bits_to_float(load_u16(w + 2));
    const uint8_t* q = w + 16;
    __m512i acc[4] = {_mm512_setzero_si512(), _mm512_setzero_si512(), _mm512_setzero_si512(), _mm512_setzero_si512()};
    int summ[4] = {0, 0, 0, 0};
    for (int j = 0; j < 4; ++j) {
      uint8_t sc0, m0, sc1, m1; get_scale_min_k4(2 * j, w + 4, &sc0, &m0); get_scale_min_k4(2 * j + 1, w + 4, &sc1, &m1);
      const __m256i qb = _mm256_loadu_si256((const __m256i*)q);
      const __m512i wv = _mm512_inserti64x4(_mm512_castsi256_si512(_mm256_and_si256(qb, m4)), _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4), 1);
      const __m512i scv = _mm512_inserti64x4(_mm512_castsi256_si512(_mm256_set1_epi32(sc0)), _mm256_set1_epi32(sc1), 1);
      for (int b = 0; b < 4; ++b) {
        const Q8K& ab = a[(int64_t)b * a_stride + i];
        const __m512i p = _mm512_dpbusd_epi32(_mm512_setzero_si512(), wv, _mm512_loadu_si512((const void*)(ab.qs + 64 * j)));
        acc[b] = _mm512_add_epi32(acc[b], _mm512_mullo_epi32(p, scv));
        summ[b] += m0 * (ab.bsums[4 * j] + ab.bsums[4 * j + 1]) + m1 * (ab.bsums[4 * j + 2] + ab.bsums[4 * j + 3]);
      }
      q += 32;
    }
    for (int b = 0; b < 4; ++b) {
      const float ad = a[(int64_t)b * a_stride + i].d;
      const float d = dw * ad, dmin = dminw * ad;
      sumf[b] = fmaf(-dmin, (float)summ[b], fmaf(d, (float)_mm512_reduce_add_epi32(acc[b]), sumf[b]));
    }
  }
  for (int b = 0; b < 4; ++b) out[b] = sumf[b];
}
// Q6_K: per 128-weight half, four 32-byte operands; (q - 32) . a = q . a - 32 * sum(a), the sums come from the Q8_K block sums
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni")))
float dot_q6k_q8k_vnni(const uint8_t* w, const Q8K* a, int nb) {
  const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3);
  float sumf = 0;
  for (int i = 0; i < nb; ++i, w += 210) {
    const uint8_t* ql = w; const uint8_t* qh = w + 128; const int8_t* sc = (const int8_t*)(w + 192);
    const float d = half_bits_to_float(load_u16(w + 208)) * a[i].d; const int8_t* q8 = a[i].qs;
    __m256i acc = _mm256_setzero_si256(); int corr = 0;
    for (int n = 0; n < 2; ++n) {
      const __m256i l0 = _mm256_loadu_si256((const __m256i*)ql), l1 = _mm256_loadu_si256((const __m256i*)(ql + 32));
      const __m256i h = _mm256_loadu_si256((const __m256i*)qh);
      __m256i q[4];
      q[0] = _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_slli_epi16(_mm256_and_si256(h, m2), 4));
      q[1] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4));
      q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4));
      q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4));
      for (int t = 0; t < 4; ++t) {
        const __m256i p = _mm256_dpbusd_epi32(_mm256_setzero_si256(), q[t], _mm256_loadu_si256((const __m256i*)(q8 + 32 * t)));
        // lanes 0..3 cover the first 16 weights (scale 2t), lanes 4..7 the second 16 (scale 2t + 1)
        const __m256i s = _mm256_set_m128i(_mm_set1_epi32(sc[2 * t + 1]), _mm_set1_epi32(sc[2 * t]));
        acc = _mm256_add_epi32(acc, _mm256_mullo_epi32(p, s));
        corr += sc[2 * t] * a[i].bsums[8 * n + 2 * t] + sc[2 * t + 1] * a[i].bsums[8 * n + 2 * t + 1];
      }
      ql += 64; qh += 32; sc += 8; q8 += 128;
    }
    sumf += d * (float)(hsum8i(acc) - 32 * corr);
  }
  return sumf;
}
bool has_avx2() { static const bool v = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); return v; }
bool has_vnni512() {
  static const bool v = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl") &&
                        __builtin_cpu_supports("avx512vnni") && !std::getenv("RLZ_NO_AVX512");
  return v;
}
#else
bool has_avx2() { return false; }
bool has_vnni512() { return false; }
#endif

float dot_legacy_q8_0(int qtype, const uint8_t* w, const Q80A* a, int nb) {
  // legacy 32-element blocks against Q8_0-quantised activations
#if RLZ_X86
  if (qtype == QT_Q8_0 || qtype == QT_Q4_0 || qtype == QT_Q5_0 || qtype == QT_Q4_1 || qtype == QT_Q5_1) {
    if (has_vnni512()) return dot_legacy_q8_0_vnni(qtype, w, a, nb);
    if (has_avx2()) return dot_legacy_q8_0_avx2(qtype, w, a, nb);
  }
#endif
  float sumf = 0; const int bb = qtype_block_bytes(qtype);
  for (int i = 0; i < nb; ++i, w += bb) {
    const float da = a[i].d; const int8_t* q8 = a[i].qs;
    switch (qtype) {
      case QT_Q4_0: {
        const float d = half_bits_to_float(load_u16(w)); int s = 0;
        for (int j = 0; j < 16; ++j) s += ((int)(w[2 + j] & 0xF) - 8) * q8[j] + ((int)(w[2 + j] >> 4) - 8) * q8[j + 16];
        sumf += d * da * s; break; }
      case QT_Q8_0: {
        const float d = half_bits_to_float(load_u16(w)); int s = 0; const int8_t* q = (const int8_t*)(w + 2);
        for (int j = 0; j < 32; ++j) s += q[j] * q8[j];
        sumf += d * da * s; break; }
      default: {
        float tmp[32]; dequant_block(qtype, w, tmp); float s = 0;
        for (int j = 0; j < 32; ++j) s += tmp[j] * (da * q8[j]);
        sumf += s; }
    }
  }
  return sumf;
}

inline bool is_kquant(int t) { return t == QT_Q4_K || t == QT_Q5_K || t == QT_Q6_K || t == QT_Q2_K; }

float dot_kquant(int qtype, const uint8_t* w, const Q8K* a, int nb) {
  switch (qtype) {
    case QT_Q4_K:
#if RLZ_X86
      if (has_vnni512()) return dot_q4k_q8k_vnni(w, a, nb);
      if (has_avx2()) return dot_q4k_q8k_avx2(w, a, nb);
#endif
      return dot_q4k_q8k_scalar(w, a, nb);
    case QT_Q5_K:
#if RLZ_X86
      if (has_avx2()) return dot_q5k_q8k_avx2(w, a, nb);
#endif
      return dot_q5k_q8k_scalar(w, a, nb);
    case QT_Q6_K:
#if RLZ_X86
      if (has_vnni512()) return dot_q6k_q8k_vnni(w, a, nb);
      if (has_avx2()) return dot_q6k_q8k_avx2(w, a, nb);
#endif
      return dot_q6k_q8k_scalar(w, a, nb);
    default: {
      float tmp[256], s = 0; const int bb = qtype_block_bytes(qtype);
      for (int i = 0; i < nb; ++i) { dequant_block(qtype, w + (int64_t)i * bb, tmp); for (int j = 0; j < 256; ++j) s += tmp[j] * (a[i].d * a[i].qs[j]); }
      return s; }
  }
}

}  // namespace

// ====================================================================== C API ========
extern "C" {

int rlz_block_elems(int qtype) { return qtype_block_elems(qtype); }
int rlz_block_bytes(int qtype) { return qtype_block_bytes(qtype); }
int rlz_cpu_threads() { return pool().size(); }
int rlz_cpu_has_avx2() { return has_avx2() ? 1 : 0; }
int rlz_cpu_has_avx512_vnni() { return has_vnni512() ? 1 : 0; }
// which code path a block type's fused dot takes on this host: 0 scalar, 1 AVX2, 2 AVX-512 VNNI
int rlz_cpu_dot_path(int qtype) {
  switch (qtype) {
    case QT_Q4_K: case QT_Q6_K: return has_vnni512() ? 2 : has_avx2() ? 1 : 0;
    case QT_Q8_0: case QT_Q4_0: case QT_Q5_0: case QT_Q4_1: case QT_Q5_1: return has_vnni512() ? 2 : has_avx2() ? 1 : 0;
    case QT_Q5_K: return has_avx2() ? 1 : 0;
    default: return 0;
  }
}

// bytes of one row of `k` elements, or -1 if k is not a multiple of the block size
int64_t rlz_row_bytes(int qtype, int64_t k) {
  const int be = qtype_block_elems(qtype);
  if (!be || k % be) return -1;
  return k / be * qtype_block_bytes(qtype);
}

// Quantise nrows x k floats (row-major) into dst.  Returns 0 on success.
int rlz_quantize(int qtype, const float* src, void* dst, int64_t nrows, int64_t k) {
  const int64_t rb = rlz_row_bytes(qtype, k);
  if (rb < 0) return -1;
  void (*fn)(const float*, uint8_t*, int64_t) = nullptr;
  switch (qtype) {
    case QT_Q4_0: fn = quantize_row_q4_0; break; case QT_Q4_1: fn = quantize_row_q4_1; break;
    case QT_Q5_0: fn = quantize_row_q5_0; break; case QT_Q5_1: fn = quantize_row_q5_1; break;
    case QT_Q8_0: fn = quantize_row_q8_0; break; case QT_Q2_K: fn = quantize_row_q2_k; break;
    case QT_Q4_K: fn = quantize_row_q4_k; break; case QT_Q5_K: fn = quantize_row_q5_k; break;
    case QT_Q6_K: fn = quantize_row_q6_k; break;
    case QT_F32: memcpy(dst, src, (size_t)(nrows * k * 4)); return 0;
    case QT_F16: { uint16_t* o = (uint16_t*)dst; for (int64_t i = 0; i < nrows * k; ++i) o[i] = float_to_half_bits(src[i]); return 0; }
    case QT_BF16: { uint16_t* o = (uint16_t*)dst; for (int64_t i = 0; i < nrows * k; ++i) o[i] = float_to_bf16_bits(src[i]); return 0; }
    default: return -2;
  }
  std::atomic<int64_t> next{0};
  pool().run([&](int) {
    for (;;) {
      int64_t r = next.fetch_add(16); if (r >= nrows) break;
      for (int64_t rr = r; rr < std::min(nrows, r + 16); ++rr) fn(src + rr * k, (uint8_t*)dst + rr * rb, k);
    }
  });
  return 0;
}

// Dequantise n elements (n multiple of the block size) to f32.
int rlz_dequantize(int qtype, const void* src, float* dst, int64_t n) {
  const int be = qtype_block_elems(qtype), bb = qtype_block_bytes(qtype);
  if (!be || n % be) return -1;
  if (qtype == QT_F32) { memcpy(dst, src, (size_t)n * 4); return 0; }
  if (qtype == QT_F16) { const uint16_t* s = (const uint16_t*)src; for (int64_t i = 0; i < n; ++i) dst[i] = half_bits_to_float(s[i]); return 0; }
  if (qtype == QT_BF16) { const uint16_t* s = (const uint16_t*)src; for (int64_t i = 0; i < n; ++i) dst[i] = bf16_bits_to_float(s[i]); return 0; }
  float probe[256];
  if (!dequant_block(qtype, (const uint8_t*)src, probe) && n > 0) return -2;
  const int64_t nb = n / be; std::atomic<int64_t> next{0};
  pool().run([&](int) {
    for (;;) {
      int64_t b0 = next.fetch_add(256); if (b0 >= nb) break;
      for (int64_t b = b0; b < std::min(nb, b0 + 256); ++b) dequant_block(qtype, (const uint8_t*)src + b * bb, dst + b * be);
    }
  });
  return 0;
}

// y[n] = W[n,k] . x[k]   (W in block layout `qtype`; x f32).  Fused dequant-dot: activations
// are quantised once (Q8_K for K-quants, Q8_0 for 32-element blocks); dense types use f32 math.
// `batch` activation rows are processed against each weight row (y is [batch, n]).
int rlz_matvec(int qtype, const void* W, const float* x, float* y, int64_t n, int64_t k, int64_t batch) {
  const int64_t rb = rlz_row_bytes(qtype, k);
  if (rb < 0) return -1;
  const uint8_t* w = (const uint8_t*)W;
  if (qtype == QT_F32 || qtype == QT_F16 || qtype == QT_BF16) {
    std::atomic<int64_t> next{0};
    pool().run([&](int) {
      for (;;) {
        int64_t r0 = next.fetch_add(8); if (r0 >= n) break;
        for (int64_t r = r0; r < std::min(n, r0 + 8); ++r)
          for (int64_t b = 0; b < batch; ++b) {
            const float* xb = x + b * k; double s = 0;
            if (qtype == QT_F32) { const float* wr = (const float*)(w + r * rb); for (int64_t j = 0; j < k; ++j) s += (double)wr[j] * xb[j]; }
            else { const uint16_t* wr = (const uint16_t*)(w + r * rb);
              for (int64_t j = 0; j < k; ++j) s += (double)(qtype == QT_F16 ? half_bits_to_float(wr[j]) : bf16_bits_to_float(wr[j])) * xb[j]; }
            y[b * n + r] = (float)s;
          }
      }
    });
    return 0;
  }
  if (is_kquant(qtype)) {
    const int nb = (int)(k / 256);
    std::vector<Q8K> act((size_t)nb * batch);
    for (int64_t b = 0; b < batch; ++b) quantize_q8_k(x + b * k, act.data() + b * nb, k);
    std::atomic<int64_t> next{0};
    pool().run([&](int) {
      for (;;) {
        int64_t r0 = next.fetch_add(32); if (r0 >= n) break;
        for (int64_t r = r0; r < std::min(n, r0 + 32); ++r) {
          int64_t b = 0;
#if RLZ_X86
          if (qtype == QT_Q4_K && has_vnni512())             // four activation rows per pass over the weight row
            for (; b + 4 <= batch; b += 4) {
              float o[4]; dot_q4k_q8k_vnni_x4(w + r * rb, act.data() + b * nb, nb, nb, o);
              for (int t = 0; t < 4; ++t) y[(b + t) * n + r] = o[t];
            }
#endif
          for (; b < batch; ++b) y[b * n + r] = dot_kquant(qtype, w + r * rb, act.data() + b * nb, nb);
        }
      }
    });
    return 0;
  }
  const int nb = (int)(k / 32);
  std::vector<Q80A> act((size_t)nb * batch);
  for (int64_t b = 0; b < batch; ++b) quantize_q8_0_act(x + b * k, act.data() + b * nb, k);
  std::atomic<int64_t> next{0};
  pool().run([&](int) {
    for (;;) {
      int64_t r0 = next.fetch_add(32); if (r0 >= n) break;
      for (int64_t r = r0; r < std::min(n, r0 + 32); ++r)
        for (int64_t b = 0; b < batch; ++b) y[b * n + r] = dot_legacy_q8_0(qtype, w + r * rb, act.data() + b * nb, nb);
    }
  });
  return 0;
}

// Several weight matrices with the same input (Q / K / V, gate / up): the activation rows are quantised once and the rows of all
// matrices are spread over the pool in ONE parallel region (a decode step of a small model is bounded by the number of such
// regions, not by their arithmetic).  All matrices must take the same activation format (all K-quants or all 32-weight block
// types); returns -2 otherwise and the caller falls back to one call per matrix.  Row by row the results equal rlz_matvec.
int rlz_matvec_multi(int nmat, const int* qtypes, const void* const* Ws, const int64_t* ns, int64_t k, const float* x, float* const* ys, int64_t batch) {
  if (nmat < 1 || nmat > 4) return -1;
  bool kq = is_kquant(qtypes[0]);
  int64_t rbs[4], starts[5] = {0, 0, 0, 0, 0};
  for (int m = 0; m < nmat; ++m) {
    const int qt = qtypes[m];
    if (qt == QT_F32 || qt == QT_F16 || qt == QT_BF16 || is_kquant(qt) != kq) return -2;
    rbs[m] = rlz_row_bytes(qt, k);
    if (rbs[m] < 0) return -1;
    starts[m + 1] = starts[m] + ns[m];
  }
  const int64_t total = starts[nmat];
  const int nb = (int)(kq ? k / 256 : k / 32);
  std::vector<Q8K> actk; std::vector<Q80A> actl;
  if (kq) { actk.resize((size_t)nb * batch); for (int64_t b = 0; b < batch; ++b) quantize_q8_k(x + b * k, actk.data() + b * nb, k); }
  else { actl.resize((size_t)nb * batch); for (int64_t b = 0; b < batch; ++b) quantize_q8_0_act(x + b * k, actl.data() + b * nb, k); }
  std::atomic<int64_t> next{0};
  pool().run([&](int) {
    for (;;) {
      int64_t g0 = next.fetch_add(32); if (g0 >= total) break;
      for (int64_t g = g0; g < std::min(total, g0 + 32); ++g) {
        int m = 0; while (g >= starts[m + 1]) ++m;
        const int64_t r = g - starts[m], n = ns[m];
        const uint8_t* wr = (const uint8_t*)Ws[m] + r * rbs[m];
        for (int64_t b = 0; b < batch; ++b)
          ys[m][b * n + r] = kq ? dot_kquant(qtypes[m], wr, actk.data() + b * nb, nb) : dot_legacy_q8_0(qtypes[m], wr, actl.data() + b * nb, nb);
      }
    }
  });
  return 0;
}

// run fn over [0,n) in parallel chunks (exposed for the CPU engine in this library)
void rlz_parallel_for(int64_t n, int64_t chunk, void (*fn)(int64_t, int64_t, void*), void* ctx) {
  std::atomic<int64_t> next{0};
  pool().run([&](int) {
    for (;;) { int64_t b = next.fetch_add(chunk); if (b >= n) break; fn(b, std::min(n, b + chunk), ctx); }
  });
}

}  // extern "C"
