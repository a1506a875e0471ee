// C++ CPU decoder: single-token forward with a KV cache over block-quantised weights.
// It is both the CPU configuration of the engine and the numerical oracle for the GPU path.
//
// Data flow per token (capability parity with the reference's CPU path,
// src/gguf/inference/forward/forward_cached.rs:11-398):
//   embed -> [+ absolute position] -> per layer { norm -> QKV(+bias) -> per-head QK-norm ->
//   RoPE (NORM/NEOX, partial rotary) -> cache append -> GQA attention -> o_proj(+bias) ->
//   residual -> FFN (SwiGLU or GELU MLP) -> residual } -> final norm -> lm_head(+bias).
// Phi-2 style parallel residual (x + attn(ln x) + mlp(ln x)) shares the single pre-norm.
#include "quant_blocks.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

using namespace rlz;

extern "C" {
int rlz_matvec(int qtype, const void* W, const float* x, float* y, int64_t n, int64_t k, int64_t batch);
int rlz_matvec_multi(int nmat, const int* qtypes, const void* const* Ws, const int64_t* ns, int64_t k, const float* x, float* const* ys, int64_t batch);
int rlz_dequantize(int qtype, const void* src, float* dst, int64_t n);
int64_t rlz_row_bytes(int qtype, int64_t k);
void rlz_parallel_for(int64_t n, int64_t chunk, void (*fn)(int64_t, int64_t, void*), void* ctx);
}

namespace {

struct Tensor { int qtype = -1; const uint8_t* data = nullptr; int64_t n = 0, k = 0; bool ok() const { return data != nullptr; } };

struct Config {
  int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, intermediate, vocab;
  int32_t rope_dim;        // rotated dims per head (<= head_dim); 0 disables RoPE
  int32_t rope_type;       // 0 = adjacent pairs (NORM), 2 = split halves (NEOX)
  int32_t norm_type;       // 0 = RMSNorm, 1 = LayerNorm
  int32_t gated_ffn;       // 1 = SwiGLU (gate,up,down), 0 = GELU MLP (up,down)
  int32_t parallel_residual;
  int32_t max_seq;
  float rope_theta, eps;
};

struct Layer {
  Tensor attn_norm_w, attn_norm_b, ffn_norm_w, ffn_norm_b;
  Tensor qkv_w, qkv_b, q_w, q_b, k_w, k_b, v_w, v_b, o_w, o_b;
  Tensor gate_w, gate_b, up_w, up_b, down_w, down_b, q_norm_w, k_norm_w;
};

struct Model {
  Config cfg;
  Tensor tok_embd, pos_embd, out_norm_w, out_norm_b, out_w, out_b;
  std::vector<Layer> layers;
  // KV cache: [layer][pos][kv_dim]
  std::vector<float> kcache, vcache;
  std::vector<float> x, h, q, k, v, qkv, att, tmp, gate, up, act, ffn, scores, logits;
  std::vector<float> trace;  // per-layer residual-stream L2 norms of the last forward
};

void vec_from(const Tensor& t, std::vector<float>& out) {
  out.resize((size_t)(t.n * t.k));
  rlz_dequantize(t.qtype, t.data, out.data(), t.n * t.k);
}

void norm(const Config& c, const float* x, float* y, int n, const Tensor& w, const Tensor& b,
          std::vector<float>& wbuf, std::vector<float>& bbuf) {
  if (w.ok() && (int)wbuf.size() != n) vec_from(w, wbuf);
  if (b.ok() && (int)bbuf.size() != n) vec_from(b, bbuf);
  if (c.norm_type == 0) {
    double ss = 0; for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
    const float inv = 1.f / sqrtf((float)(ss / n) + c.eps);
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv * (w.ok() ? wbuf[i] : 1.f);
  } else {
    double mean = 0; for (int i = 0; i < n; ++i) mean += x[i]; mean /= n;
    double var = 0; for (int i = 0; i < n; ++i) { double d = x[i] - mean; var += d * d; } var /= n;
    const float inv = 1.f / sqrtf((float)var + c.eps);
    for (int i = 0; i < n; ++i) y[i] = (float)(x[i] - mean) * inv * (w.ok() ? wbuf[i] : 1.f) + (b.ok() ? bbuf[i] : 0.f);
  }
}

struct NormCache { std::vector<float> w, b; };

void linear(const Tensor& w, const Tensor& b, const float* x, float* y, std::vector<float>& bbuf) {
  rlz_matvec(w.qtype, w.data, x, y, w.n, w.k, 1);
  if (b.ok()) {
    if ((int64_t)bbuf.size() != w.n) vec_from(b, bbuf);
    for (int64_t i = 0; i < w.n; ++i) y[i] += bbuf[i];
  }
}

// Up to three projections of the same input in one parallel region (falls back to one region each when their block types need
// different activation formats); biases are added afterwards.  T rows of x ([T, k]) give T rows per output ([T, n]).
struct Proj { const Tensor* w; const Tensor* b; float* y; std::vector<float>* bbuf; };
void linear_group(Proj* ps, int np, const float* x, int T) {
  int qts[4]; const void* Ws[4]; int64_t ns[4]; float* ys[4];
  for (int i = 0; i < np; ++i) { qts[i] = ps[i].w->qtype; Ws[i] = ps[i].w->data; ns[i] = ps[i].w->n; ys[i] = ps[i].y; }
  bool same_k = true; for (int i = 1; i < np; ++i) same_k &= ps[i].w->k == ps[0].w->k;
  if (!same_k || np < 2 || rlz_matvec_multi(np, qts, Ws, ns, ps[0].w->k, x, ys, T) != 0)
    for (int i = 0; i < np; ++i) rlz_matvec(qts[i], Ws[i], x, ys[i], ns[i], ps[i].w->k, T);
  for (int i = 0; i < np; ++i) {
    const Tensor& b = *ps[i].b;
    if (!b.ok()) continue;
    if ((int64_t)ps[i].bbuf->size() != ns[i]) vec_from(b, *ps[i].bbuf);
    for (int t = 0; t < T; ++t) for (int64_t j = 0; j < ns[i]; ++j) ys[i][(size_t)t * ns[i] + j] += (*ps[i].bbuf)[j];
  }
}

// (cos, sin) of every rotary pair at one position: computed once per token and shared by all layers and heads
void rope_table(const Config& c, int pos, std::vector<float>& cs) {
  const int rd = c.rope_dim, half = rd / 2;
  cs.resize(rd > 0 ? (size_t)2 * half : 0);
  for (int i = 0; i < half; ++i) {
    const float freq = powf(c.rope_theta, -2.f * i / rd);
    const float ang = pos * freq;
    cs[2 * i] = cosf(ang); cs[2 * i + 1] = sinf(ang);
  }
}

void rope(const Config& c, float* v, int n_heads, const std::vector<float>& cs_tab) {
  const int rd = c.rope_dim; if (rd <= 0) return;
  const int half = rd / 2;
  for (int h = 0; h < n_heads; ++h) {
    float* p = v + (size_t)h * c.head_dim;
    for (int i = 0; i < half; ++i) {
      const float cs = cs_tab[2 * i], sn = cs_tab[2 * i + 1];
      const int i0 = c.rope_type == 2 ? i : 2 * i, i1 = c.rope_type == 2 ? i + half : 2 * i + 1;
      const float a = p[i0], b = p[i1];
      p[i0] = a * cs - b * sn; p[i1] = a * sn + b * cs;
    }
  }
}

void head_rmsnorm(const Config& c, float* v, int n_heads, const std::vector<float>& w) {
  for (int h = 0; h < n_heads; ++h) {
    float* p = v + (size_t)h * c.head_dim; double ss = 0;
    for (int i = 0; i < c.head_dim; ++i) ss += (double)p[i] * p[i];
    const float inv = 1.f / sqrtf((float)(ss / c.head_dim) + c.eps);
    for (int i = 0; i < c.head_dim; ++i) p[i] = p[i] * inv * w[i];
  }
}

inline float gelu_tanh(float x) { return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x))); }
inline float silu(float x) { return x / (1.f + expf(-x)); }

struct AttnCtx { Model* m; int layer; int pos; };

void attn_heads(int64_t h0, int64_t h1, void* vp) {
  AttnCtx* a = (AttnCtx*)vp; Model& m = *a->m; const Config& c = m.cfg;
  const int kv_dim = c.n_kv_heads * c.head_dim, group = c.n_heads / c.n_kv_heads, len = a->pos + 1;
  const float scale = 1.f / sqrtf((float)c.head_dim);
  const float* kc = m.kcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
  const float* vc = m.vcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
  for (int64_t h = h0; h < h1; ++h) {
    const int kvh = (int)h / group; const float* qh = m.q.data() + h * c.head_dim;
    float* sc = m.scores.data() + (size_t)h * c.max_seq; float mx = -INFINITY;
    for (int t = 0; t < len; ++t) {
      const float* kr = kc + (size_t)t * kv_dim + kvh * c.head_dim; float s = 0;
      for (int i = 0; i < c.head_dim; ++i) s += qh[i] * kr[i];
      sc[t] = s * scale; mx = std::max(mx, sc[t]);
    }
    float sum = 0; for (int t = 0; t < len; ++t) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
    float* o = m.att.data() + h * c.head_dim; for (int i = 0; i < c.head_dim; ++i) o[i] = 0;
    for (int t = 0; t < len; ++t) {
      const float* vr = vc + (size_t)t * kv_dim + kvh * c.head_dim; const float p = sc[t] / sum;
      for (int i = 0; i < c.head_dim; ++i) o[i] += p * vr[i];
    }
  }
}

struct Runtime {
  std::vector<NormCache> attn_nc, ffn_nc; NormCache out_nc;
  std::vector<std::vector<float>> qkv_b, q_b, k_b, v_b, o_b, gate_b, up_b, down_b, qn, kn;
  std::vector<float> out_b;
};
std::map<Model*, Runtime> g_rt;

int forward(Model& m, int token, int pos, float* logits_out) {
  const Config& c = m.cfg; Runtime& rt = g_rt[&m];
  if (pos < 0 || pos >= c.max_seq || token < 0 || token >= c.vocab) return -1;
  const int H = c.hidden, qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
  // embedding row (dequantised per row)
  { const int64_t rb = rlz_row_bytes(m.tok_embd.qtype, H); if (rb < 0) return -2;
    rlz_dequantize(m.tok_embd.qtype, m.tok_embd.data + (int64_t)token * rb, m.x.data(), H); }
  if (m.pos_embd.ok()) {
    const int64_t rb = rlz_row_bytes(m.pos_embd.qtype, H);
    rlz_dequantize(m.pos_embd.qtype, m.pos_embd.data + (int64_t)pos * rb, m.tmp.data(), H);
    for (int i = 0; i < H; ++i) m.x[i] += m.tmp[i];
  }
  m.trace.assign(c.n_layers, 0.f);
  std::vector<float> cs_tab; rope_table(c, pos, cs_tab);
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = m.layers[l];
    norm(c, m.x.data(), m.h.data(), H, L.attn_norm_w, L.attn_norm_b, rt.attn_nc[l].w, rt.attn_nc[l].b);
    if (L.qkv_w.ok()) {
      linear(L.qkv_w, L.qkv_b, m.h.data(), m.qkv.data(), rt.qkv_b[l]);
      std::copy(m.qkv.begin(), m.qkv.begin() + qd, m.q.begin());
      std::copy(m.qkv.begin() + qd, m.qkv.begin() + qd + kvd, m.k.begin());
      std::copy(m.qkv.begin() + qd + kvd, m.qkv.begin() + qd + 2 * kvd, m.v.begin());
    } else {
      Proj qkv3[3] = {{&L.q_w, &L.q_b, m.q.data(), &rt.q_b[l]}, {&L.k_w, &L.k_b, m.k.data(), &rt.k_b[l]}, {&L.v_w, &L.v_b, m.v.data(), &rt.v_b[l]}};
      linear_group(qkv3, 3, m.h.data(), 1);
    }
    if (L.q_norm_w.ok()) { if (rt.qn[l].empty()) vec_from(L.q_norm_w, rt.qn[l]); head_rmsnorm(c, m.q.data(), c.n_heads, rt.qn[l]); }
    if (L.k_norm_w.ok()) { if (rt.kn[l].empty()) vec_from(L.k_norm_w, rt.kn[l]); head_rmsnorm(c, m.k.data(), c.n_kv_heads, rt.kn[l]); }
    rope(c, m.q.data(), c.n_heads, cs_tab); rope(c, m.k.data(), c.n_kv_heads, cs_tab);
    std::copy(m.k.begin(), m.k.begin() + kvd, m.kcache.begin() + ((size_t)l * c.max_seq + pos) * kvd);
    std::copy(m.v.begin(), m.v.begin() + kvd, m.vcache.begin() + ((size_t)l * c.max_seq + pos) * kvd);
    AttnCtx actx{&m, l, pos};
    rlz_parallel_for(c.n_heads, 1, attn_heads, &actx);
    linear(L.o_w, L.o_b, m.att.data(), m.tmp.data(), rt.o_b[l]);
    const float* ffn_in;
    if (c.parallel_residual) { ffn_in = m.h.data(); }
    else {
      for (int i = 0; i < H; ++i) m.x[i] += m.tmp[i];
      norm(c, m.x.data(), m.h.data(), H, L.ffn_norm_w, L.ffn_norm_b, rt.ffn_nc[l].w, rt.ffn_nc[l].b);
      ffn_in = m.h.data();
    }
    if (c.gated_ffn) {
      Proj gu[2] = {{&L.gate_w, &L.gate_b, m.gate.data(), &rt.gate_b[l]}, {&L.up_w, &L.up_b, m.up.data(), &rt.up_b[l]}};
      linear_group(gu, 2, ffn_in, 1);
      for (int i = 0; i < c.intermediate; ++i) m.act[i] = silu(m.gate[i]) * m.up[i];
    } else {
      linear(L.up_w, L.up_b, ffn_in, m.up.data(), rt.up_b[l]);
      for (int i = 0; i < c.intermediate; ++i) m.act[i] = gelu_tanh(m.up[i]);
    }
    linear(L.down_w, L.down_b, m.act.data(), m.ffn.data(), rt.down_b[l]);
    if (c.parallel_residual) for (int i = 0; i < H; ++i) m.x[i] += m.tmp[i] + m.ffn[i];
    else for (int i = 0; i < H; ++i) m.x[i] += m.ffn[i];
    double ss = 0; for (int i = 0; i < H; ++i) ss += (double)m.x[i] * m.x[i];
    m.trace[l] = (float)sqrt(ss);
  }
  norm(c, m.x.data(), m.h.data(), H, m.out_norm_w, m.out_norm_b, rt.out_nc.w, rt.out_nc.b);
  linear(m.out_w, m.out_b, m.h.data(), m.logits.data(), rt.out_b);
  if (logits_out) std::copy(m.logits.begin(), m.logits.end(), logits_out);
  return 0;
}

// ---- prompt chunks: T consecutive tokens of one sequence in one pass --------------------------------------------------------
// Every projection runs as ONE batched matrix-vector product (each weight row is read once and multiplied with the T quantised
// activation rows), attention runs per (token, head) over the cache up to the token's own position, and only the last token
// goes through the output matrix.  Row by row the arithmetic is the same as in forward(), so the logits of the last token are
// bit-identical to a token-by-token prompt.  (Role of the reference's batched CPU prefill: append_kv / advance_by,
// src/gguf/runtime.rs:123-298.)
struct ChunkCtx { Model* m; int layer, pos0, T; const float* q; float* att; float* scores; };

void attn_chunk(int64_t j0, int64_t j1, void* vp) {
  ChunkCtx* a = (ChunkCtx*)vp; Model& m = *a->m; const Config& c = m.cfg;
  const int kv_dim = c.n_kv_heads * c.head_dim, group = c.n_heads / c.n_kv_heads, qd = c.n_heads * c.head_dim;
  const float scale = 1.f / sqrtf((float)c.head_dim);
  const float* kc = m.kcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
  const float* vc = m.vcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
  for (int64_t j = j0; j < j1; ++j) {                      // job = (token, head)
    const int t = (int)(j / c.n_heads), h = (int)(j % c.n_heads), len = a->pos0 + t + 1, kvh = h / group;
    const float* qh = a->q + (size_t)t * qd + (size_t)h * c.head_dim;
    float* sc = a->scores + (size_t)j * c.max_seq; float mx = -INFINITY;
    for (int u = 0; u < len; ++u) {
      const float* kr = kc + (size_t)u * kv_dim + kvh * c.head_dim; float s = 0;
      for (int i = 0; i < c.head_dim; ++i) s += qh[i] * kr[i];
      sc[u] = s * scale; mx = std::max(mx, sc[u]);
    }
    float sum = 0; for (int u = 0; u < len; ++u) { sc[u] = expf(sc[u] - mx); sum += sc[u]; }
    float* o = a->att + (size_t)t * qd + (size_t)h * c.head_dim; for (int i = 0; i < c.head_dim; ++i) o[i] = 0;
    for (int u = 0; u < len; ++u) {
      const float* vr = vc + (size_t)u * kv_dim + kvh * c.head_dim; const float p = sc[u] / sum;
      for (int i = 0; i < c.head_dim; ++i) o[i] += p * vr[i];
    }
  }
}

void linear_rows(const Tensor& w, const Tensor& b, const float* x, float* y, int T, std::vector<float>& bbuf) {
  rlz_matvec(w.qtype, w.data, x, y, w.n, w.k, T);
  if (b.ok()) {
    if ((int64_t)bbuf.size() != w.n) vec_from(b, bbuf);
    for (int t = 0; t < T; ++t) for (int64_t i = 0; i < w.n; ++i) y[(size_t)t * w.n + i] += bbuf[i];
  }
}

int forward_chunk(Model& m, const int* tokens, int T, int pos0, float* logits_out) {
  const Config& c = m.cfg; Runtime& rt = g_rt[&m];
  if (T < 1 || pos0 < 0 || pos0 + T > c.max_seq) return -1;
  const int H = c.hidden, qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim, I = c.intermediate;
  std::vector<float> x((size_t)T * H), h((size_t)T * H), q((size_t)T * qd), k((size_t)T * kvd), v((size_t)T * kvd), qkv, att((size_t)T * qd),
      tmp((size_t)T * H), up((size_t)T * I), gate, act((size_t)T * I), ffn((size_t)T * H), scores((size_t)T * c.n_heads * c.max_seq), row(H);
  for (int t = 0; t < T; ++t) {
    if (tokens[t] < 0 || tokens[t] >= c.vocab) return -1;
    const int64_t rb = rlz_row_bytes(m.tok_embd.qtype, H); if (rb < 0) return -2;
    rlz_dequantize(m.tok_embd.qtype, m.tok_embd.data + (int64_t)tokens[t] * rb, x.data() + (size_t)t * H, H);
    if (m.pos_embd.ok()) {
      const int64_t pb = rlz_row_bytes(m.pos_embd.qtype, H);
      rlz_dequantize(m.pos_embd.qtype, m.pos_embd.data + (int64_t)(pos0 + t) * pb, row.data(), H);
      for (int i = 0; i < H; ++i) x[(size_t)t * H + i] += row[i];
    }
  }
  if (c.gated_ffn) gate.resize((size_t)T * I);
  std::vector<std::vector<float>> cs_tabs(T);
  for (int t = 0; t < T; ++t) rope_table(c, pos0 + t, cs_tabs[t]);
  m.trace.assign(c.n_layers, 0.f);
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = m.layers[l];
    for (int t = 0; t < T; ++t) norm(c, x.data() + (size_t)t * H, h.data() + (size_t)t * H, H, L.attn_norm_w, L.attn_norm_b, rt.attn_nc[l].w, rt.attn_nc[l].b);
    if (L.qkv_w.ok()) {
      qkv.resize((size_t)T * (qd + 2 * kvd));
      linear_rows(L.qkv_w, L.qkv_b, h.data(), qkv.data(), T, rt.qkv_b[l]);
      for (int t = 0; t < T; ++t) {
        const float* r = qkv.data() + (size_t)t * (qd + 2 * kvd);
        std::copy(r, r + qd, q.begin() + (size_t)t * qd);
        std::copy(r + qd, r + qd + kvd, k.begin() + (size_t)t * kvd);
        std::copy(r + qd + kvd, r + qd + 2 * kvd, v.begin() + (size_t)t * kvd);
      }
    } else {
      Proj qkv3[3] = {{&L.q_w, &L.q_b, q.data(), &rt.q_b[l]}, {&L.k_w, &L.k_b, k.data(), &rt.k_b[l]}, {&L.v_w, &L.v_b, v.data(), &rt.v_b[l]}};
      linear_group(qkv3, 3, h.data(), T);
    }
    if (L.q_norm_w.ok() && rt.qn[l].empty()) vec_from(L.q_norm_w, rt.qn[l]);
    if (L.k_norm_w.ok() && rt.kn[l].empty()) vec_from(L.k_norm_w, rt.kn[l]);
    for (int t = 0; t < T; ++t) {
      float* qt = q.data() + (size_t)t * qd; float* kt = k.data() + (size_t)t * kvd;
      if (L.q_norm_w.ok()) head_rmsnorm(c, qt, c.n_heads, rt.qn[l]);
      if (L.k_norm_w.ok()) head_rmsnorm(c, kt, c.n_kv_heads, rt.kn[l]);
      rope(c, qt, c.n_heads, cs_tabs[t]); rope(c, kt, c.n_kv_heads, cs_tabs[t]);
      std::copy(kt, kt + kvd, m.kcache.begin() + ((size_t)l * c.max_seq + pos0 + t) * kvd);
      std::copy(v.begin() + (size_t)t * kvd, v.begin() + (size_t)(t + 1) * kvd, m.vcache.begin() + ((size_t)l * c.max_seq + pos0 + t) * kvd);
    }
    ChunkCtx actx{&m, l, pos0, T, q.data(), att.data(), scores.data()};
    rlz_parallel_for((int64_t)T * c.n_heads, 1, attn_chunk, &actx);
    linear_rows(L.o_w, L.o_b, att.data(), tmp.data(), T, rt.o_b[l]);
    if (!c.parallel_residual) {
      for (size_t i = 0; i < (size_t)T * H; ++i) x[i] += tmp[i];
      for (int t = 0; t < T; ++t) norm(c, x.data() + (size_t)t * H, h.data() + (size_t)t * H, H, L.ffn_norm_w, L.ffn_norm_b, rt.ffn_nc[l].w, rt.ffn_nc[l].b);
    }
    if (c.gated_ffn) {
      Proj gu[2] = {{&L.gate_w, &L.gate_b, gate.data(), &rt.gate_b[l]}, {&L.up_w, &L.up_b, up.data(), &rt.up_b[l]}};
      linear_group(gu, 2, h.data(), T);
      for (size_t i = 0; i < (size_t)T * I; ++i) act[i] = silu(gate[i]) * up[i];
    } else {
      linear_rows(L.up_w, L.up_b, h.data(), up.data(), T, rt.up_b[l]);
      for (size_t i = 0; i < (size_t)T * I; ++i) act[i] = gelu_tanh(up[i]);
    }
    linear_rows(L.down_w, L.down_b, act.data(), ffn.data(), T, rt.down_b[l]);
    if (c.parallel_residual) for (size_t i = 0; i < (size_t)T * H; ++i) x[i] += tmp[i] + ffn[i];
    else for (size_t i = 0; i < (size_t)T * H; ++i) x[i] += ffn[i];
    double ss = 0; const float* last = x.data() + (size_t)(T - 1) * H; for (int i = 0; i < H; ++i) ss += (double)last[i] * last[i];
    m.trace[l] = (float)sqrt(ss);
  }
  // only the last token needs logits
  std::copy(x.begin() + (size_t)(T - 1) * H, x.end(), m.x.begin());
  norm(c, m.x.data(), m.h.data(), H, m.out_norm_w, m.out_norm_b, rt.out_nc.w, rt.out_nc.b);
  linear(m.out_w, m.out_b, m.h.data(), m.logits.data(), rt.out_b);
  if (logits_out) std::copy(m.logits.begin(), m.logits.end(), logits_out);
  return 0;
}

// ---- one decode step for several sequences in lock-step --------------------------------------------------------------------
// Row r is sequence `ms[r]` (its own KV cache) fed token `tokens[r]` at position `pos[r]`; all sequences share the weights of
// ms[0] (the handles were bound to the same tensors).  Every projection, the output matrix included, is ONE batched product over
// the R rows, so a step reads the weights once whatever the number of sequences; attention runs per (row, head) on the row's own
// cache.  Row by row the arithmetic equals forward().
struct RowsCtx { Model** ms; const int* pos; int layer, R; const float* q; float* att; float* scores; };

void attn_rows(int64_t j0, int64_t j1, void* vp) {
  RowsCtx* a = (RowsCtx*)vp; const Config& c = a->ms[0]->cfg;
  const int kv_dim = c.n_kv_heads * c.head_dim, group = c.n_heads / c.n_kv_heads, qd = c.n_heads * c.head_dim;
  const float scale = 1.f / sqrtf((float)c.head_dim);
  for (int64_t j = j0; j < j1; ++j) {
    const int r = (int)(j / c.n_heads), h = (int)(j % c.n_heads), len = a->pos[r] + 1, kvh = h / group;
    Model& m = *a->ms[r];
    const float* kc = m.kcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
    const float* vc = m.vcache.data() + (size_t)a->layer * c.max_seq * kv_dim;
    const float* qh = a->q + (size_t)r * qd + (size_t)h * c.head_dim;
    float* sc = a->scores + (size_t)j * c.max_seq; float mx = -INFINITY;
    for (int u = 0; u < len; ++u) {
      const float* kr = kc + (size_t)u * kv_dim + kvh * c.head_dim; float s = 0;
      for (int i = 0; i < c.head_dim; ++i) s += qh[i] * kr[i];
      sc[u] = s * scale; mx = std::max(mx, sc[u]);
    }
    float sum = 0; for (int u = 0; u < len; ++u) { sc[u] = expf(sc[u] - mx); sum += sc[u]; }
    float* o = a->att + (size_t)r * qd + (size_t)h * c.head_dim; for (int i = 0; i < c.head_dim; ++i) o[i] = 0;
    for (int u = 0; u < len; ++u) {
      const float* vr = vc + (size_t)u * kv_dim + kvh * c.head_dim; const float p = sc[u] / sum;
      for (int i = 0; i < c.head_dim; ++i) o[i] += p * vr[i];
    }
  }
}

int forward_rows(Model** ms, const int* tokens, const int* pos, int R, float* logits_out) {
  Model& m = *ms[0]; const Config& c = m.cfg; Runtime& rt = g_rt[&m];
  if (R < 1) return -1;
  for (int r = 0; r < R; ++r) {
    const Config& cr = ms[r]->cfg;
    if (cr.hidden != c.hidden || cr.n_layers != c.n_layers || cr.max_seq != c.max_seq || cr.vocab != c.vocab) return -4;
    if (pos[r] < 0 || pos[r] >= c.max_seq || tokens[r] < 0 || tokens[r] >= c.vocab) return -1;
  }
  const int H = c.hidden, qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim, I = c.intermediate;
  std::vector<float> x((size_t)R * H), h((size_t)R * H), q((size_t)R * qd), k((size_t)R * kvd), v((size_t)R * kvd), qkv, att((size_t)R * qd),
      tmp((size_t)R * H), up((size_t)R * I), gate, act((size_t)R * I), ffn((size_t)R * H), scores((size_t)R * c.n_heads * c.max_seq), row(H);
  for (int r = 0; r < R; ++r) {
    const int64_t rb = rlz_row_bytes(m.tok_embd.qtype, H); if (rb < 0) return -2;
    rlz_dequantize(m.tok_embd.qtype, m.tok_embd.data + (int64_t)tokens[r] * rb, x.data() + (size_t)r * H, H);
    if (m.pos_embd.ok()) {
      const int64_t pb = rlz_row_bytes(m.pos_embd.qtype, H);
      rlz_dequantize(m.pos_embd.qtype, m.pos_embd.data + (int64_t)pos[r] * pb, row.data(), H);
      for (int i = 0; i < H; ++i) x[(size_t)r * H + i] += row[i];
    }
  }
  if (c.gated_ffn) gate.resize((size_t)R * I);
  std::vector<std::vector<float>> cs_tabs(R);
  for (int r = 0; r < R; ++r) rope_table(c, pos[r], cs_tabs[r]);
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = m.layers[l];
    for (int r = 0; r < R; ++r) norm(c, x.data() + (size_t)r * H, h.data() + (size_t)r * H, H, L.attn_norm_w, L.attn_norm_b, rt.attn_nc[l].w, rt.attn_nc[l].b);
    if (L.qkv_w.ok()) {
      qkv.resize((size_t)R * (qd + 2 * kvd));
      linear_rows(L.qkv_w, L.qkv_b, h.data(), qkv.data(), R, rt.qkv_b[l]);
      for (int r = 0; r < R; ++r) {
        const float* s0 = qkv.data() + (size_t)r * (qd + 2 * kvd);
        std::copy(s0, s0 + qd, q.begin() + (size_t)r * qd);
        std::copy(s0 + qd, s0 + qd + kvd, k.begin() + (size_t)r * kvd);
        std::copy(s0 + qd + kvd, s0 + qd + 2 * kvd, v.begin() + (size_t)r * kvd);
      }
    } else {
      Proj qkv3[3] = {{&L.q_w, &L.q_b, q.data(), &rt.q_b[l]}, {&L.k_w, &L.k_b, k.data(), &rt.k_b[l]}, {&L.v_w, &L.v_b, v.data(), &rt.v_b[l]}};
      linear_group(qkv3, 3, h.data(), R);
    }
    if (L.q_norm_w.ok() && rt.qn[l].empty()) vec_from(L.q_norm_w, rt.qn[l]);
    if (L.k_norm_w.ok() && rt.kn[l].empty()) vec_from(L.k_norm_w, rt.kn[l]);
    for (int r = 0; r < R; ++r) {
      float* qt = q.data() + (size_t)r * qd; float* kt = k.data() + (size_t)r * kvd; Model& mr = *ms[r];
      if (L.q_norm_w.ok()) head_rmsnorm(c, qt, c.n_heads, rt.qn[l]);
      if (L.k_norm_w.ok()) head_rmsnorm(c, kt, c.n_kv_heads, rt.kn[l]);
      rope(c, qt, c.n_heads, cs_tabs[r]); rope(c, kt, c.n_kv_heads, cs_tabs[r]);
      std::copy(kt, kt + kvd, mr.kcache.begin() + ((size_t)l * c.max_seq + pos[r]) * kvd);
      std::copy(v.begin() + (size_t)r * kvd, v.begin() + (size_t)(r + 1) * kvd, mr.vcache.begin() + ((size_t)l * c.max_seq + pos[r]) * kvd);
    }
    RowsCtx actx{ms, pos, l, R, q.data(), att.data(), scores.data()};
    rlz_parallel_for((int64_t)R * c.n_heads, 1, attn_rows, &actx);
    linear_rows(L.o_w, L.o_b, att.data(), tmp.data(), R, rt.o_b[l]);
    if (!c.parallel_residual) {
      for (size_t i = 0; i < (size_t)R * H; ++i) x[i] += tmp[i];
      for (int r = 0; r < R; ++r) norm(c, x.data() + (size_t)r * H, h.data() + (size_t)r * H, H, L.ffn_norm_w, L.ffn_norm_b, rt.ffn_nc[l].w, rt.ffn_nc[l].b);
    }
    if (c.gated_ffn) {
      Proj gu[2] = {{&L.gate_w, &L.gate_b, gate.data(), &rt.gate_b[l]}, {&L.up_w, &L.up_b, up.data(), &rt.up_b[l]}};
      linear_group(gu, 2, h.data(), R);
      for (size_t i = 0; i < (size_t)R * I; ++i) act[i] = silu(gate[i]) * up[i];
    } else {
      linear_rows(L.up_w, L.up_b, h.data(), up.data(), R, rt.up_b[l]);
      for (size_t i = 0; i < (size_t)R * I; ++i) act[i] = gelu_tanh(up[i]);
    }
    linear_rows(L.down_w, L.down_b, act.data(), ffn.data(), R, rt.down_b[l]);
    if (c.parallel_residual) for (size_t i = 0; i < (size_t)R * H; ++i) x[i] += tmp[i] + ffn[i];
    else for (size_t i = 0; i < (size_t)R * H; ++i) x[i] += ffn[i];
  }
  for (int r = 0; r < R; ++r) norm(c, x.data() + (size_t)r * H, h.data() + (size_t)r * H, H, m.out_norm_w, m.out_norm_b, rt.out_nc.w, rt.out_nc.b);
  linear_rows(m.out_w, m.out_b, h.data(), logits_out, R, rt.out_b);      // [R, vocab]
  return 0;
}

}  // namespace

extern "C" {

// cfg: 13 int32 followed by 2 float (see struct Config)
void* rlz_cpu_model_create(const void* cfg_bytes) {
  Model* m = new Model();
  memcpy(&m->cfg, cfg_bytes, sizeof(Config));
  const Config& c = m->cfg;
  m->layers.resize(c.n_layers);
  const size_t kv = (size_t)c.n_layers * c.max_seq * c.n_kv_heads * c.head_dim;
  m->kcache.assign(kv, 0.f); m->vcache.assign(kv, 0.f);
  const int qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
  m->x.resize(c.hidden); m->h.resize(c.hidden); m->tmp.resize(std::max(c.hidden, qd)); m->ffn.resize(c.hidden);
  m->q.resize(qd); m->k.resize(kvd); m->v.resize(kvd); m->qkv.resize(qd + 2 * kvd); m->att.resize(qd);
  m->gate.resize(c.intermediate); m->up.resize(c.intermediate); m->act.resize(c.intermediate);
  m->scores.resize((size_t)c.n_heads * c.max_seq); m->logits.resize(c.vocab);
  Runtime& rt = g_rt[m];
  rt.attn_nc.resize(c.n_layers); rt.ffn_nc.resize(c.n_layers);
  for (auto* v : {&rt.qkv_b, &rt.q_b, &rt.k_b, &rt.v_b, &rt.o_b, &rt.gate_b, &rt.up_b, &rt.down_b, &rt.qn, &rt.kn}) v->resize(c.n_layers);
  return m;
}

void rlz_cpu_model_free(void* mp) { Model* m = (Model*)mp; g_rt.erase(m); delete m; }

// Bind a tensor by GGUF name.  `data` is borrowed and must outlive the model.
int rlz_cpu_model_set_tensor(void* mp, const char* name, int qtype, const void* data, int64_t n, int64_t k) {
  Model& m = *(Model*)mp; Tensor t; t.qtype = qtype; t.data = (const uint8_t*)data; t.n = n; t.k = k;
  std::string s(name);
  if (s == "token_embd.weight") { m.tok_embd = t; return 0; }
  if (s == "token_pos_embd.weight") { m.pos_embd = t; return 0; }
  if (s == "output_norm.weight") { m.out_norm_w = t; return 0; }
  if (s == "output_norm.bias") { m.out_norm_b = t; return 0; }
  if (s == "output.weight") { m.out_w = t; return 0; }
  if (s == "output.bias") { m.out_b = t; return 0; }
  int l = -1; char rest[96];
  if (sscanf(name, "blk.%d.%95s", &l, rest) != 2 || l < 0 || l >= (int)m.layers.size()) return -1;
  Layer& L = m.layers[l]; std::string r(rest);
  struct { const char* n; Tensor* t; } tab[] = {
    {"attn_norm.weight", &L.attn_norm_w}, {"attn_norm.bias", &L.attn_norm_b}, {"ffn_norm.weight", &L.ffn_norm_w}, {"ffn_norm.bias", &L.ffn_norm_b},
    {"attn_qkv.weight", &L.qkv_w}, {"attn_qkv.bias", &L.qkv_b}, {"attn_q.weight", &L.q_w}, {"attn_q.bias", &L.q_b},
    {"attn_k.weight", &L.k_w}, {"attn_k.bias", &L.k_b}, {"attn_v.weight", &L.v_w}, {"attn_v.bias", &L.v_b},
    {"attn_output.weight", &L.o_w}, {"attn_output.bias", &L.o_b}, {"ffn_gate.weight", &L.gate_w}, {"ffn_gate.bias", &L.gate_b},
    {"ffn_up.weight", &L.up_w}, {"ffn_up.bias", &L.up_b}, {"ffn_down.weight", &L.down_w}, {"ffn_down.bias", &L.down_b},
    {"attn_q_norm.weight", &L.q_norm_w}, {"attn_k_norm.weight", &L.k_norm_w}};
  for (auto& e : tab) if (r == e.n) { *e.t = t; return 0; }
  return -2;
}

// 0 if every tensor the architecture needs is bound
int rlz_cpu_model_validate(void* mp) {
  Model& m = *(Model*)mp; const Config& c = m.cfg;
  if (!m.tok_embd.ok() || !m.out_w.ok()) return -1;
  for (auto& L : m.layers) {
    if (!(L.qkv_w.ok() || (L.q_w.ok() && L.k_w.ok() && L.v_w.ok()))) return -2;
    if (!L.o_w.ok() || !L.up_w.ok() || !L.down_w.ok()) return -3;
    if (c.gated_ffn && !L.gate_w.ok()) return -4;
  }
  return 0;
}

int rlz_cpu_forward(void* mp, int token, int pos, float* logits_out) { return forward(*(Model*)mp, token, pos, logits_out); }

// Prompt tokens `tokens[0..n)` at positions pos0.. in chunks of up to `chunk` tokens (each projection one batched product per
// chunk); `logits_out` receives the logits after the last token.
int rlz_cpu_prefill(void* mp, const int* tokens, int n, int pos0, int chunk, float* logits_out) {
  Model& m = *(Model*)mp;
  if (n < 1) return -1;
  if (chunk < 1) chunk = 32;
  for (int i = 0; i < n; i += chunk) {
    const int T = std::min(chunk, n - i);
    const int rc = forward_chunk(m, tokens + i, T, pos0 + i, i + T >= n ? logits_out : nullptr);
    if (rc) return rc;
  }
  return 0;
}

// One decode step for `n` sequences in lock-step: handle i is fed tokens[i] at positions[i]; logits_out is [n, vocab].
// The handles must have been bound to the same weight tensors (the weights of handle 0 are used for all rows).
int rlz_cpu_forward_rows(void** handles, const int* tokens, const int* positions, int n, float* logits_out) {
  if (n < 1 || n > 64) return -1;
  Model* ms[64];
  for (int i = 0; i < n; ++i) { ms[i] = (Model*)handles[i]; if (!ms[i]) return -1; for (int j = 0; j < i; ++j) if (ms[j] == ms[i]) return -5; }
  return forward_rows(ms, tokens, positions, n, logits_out);
}

int rlz_cpu_layer_trace(void* mp, float* out) { Model& m = *(Model*)mp; std::copy(m.trace.begin(), m.trace.end(), out); return (int)m.trace.size(); }

// Greedy generation: the prompt in chunks of 32 tokens, then n_gen argmax decode steps.
// timings[0] = prefill seconds, timings[1] = decode seconds.  Returns tokens generated.
int rlz_cpu_generate_greedy(void* mp, const int* prompt, int n_prompt, int n_gen, int eos, int* out, double* timings) {
  Model& m = *(Model*)mp; const Config& c = m.cfg;
  if (n_prompt <= 0 || n_prompt + n_gen > c.max_seq) return -1;
  auto t0 = std::chrono::steady_clock::now();
  if (rlz_cpu_prefill(mp, prompt, n_prompt, 0, 32, nullptr)) return -2;
  auto t1 = std::chrono::steady_clock::now();
  int produced = 0;
  for (int g = 0; g < n_gen; ++g) {
    int best = 0; for (int i = 1; i < c.vocab; ++i) if (m.logits[i] > m.logits[best]) best = i;
    out[produced++] = best;
    if (best == eos) break;
    if (g + 1 < n_gen) if (forward(m, best, n_prompt + g, nullptr)) return -3;
  }
  auto t2 = std::chrono::steady_clock::now();
  if (timings) { timings[0] = std::chrono::duration<double>(t1 - t0).count(); timings[1] = std::chrono::duration<double>(t2 - t1).count(); }
  return produced;
}

}  // extern "C"
