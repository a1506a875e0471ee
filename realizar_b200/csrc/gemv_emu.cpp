// Host emulation of the GPU decode GEMV: runs the very same unit functions the kernel runs
// (csrc/gemv_units.h) over weights in the device layout, so the bit manipulation of every
// fast-path block type is verifiable without a GPU.
#include "gemv_blocks.h"

#include <vector>

using namespace rlz;

namespace {
template <int QT>
void emu_rows(const uint8_t* W, int64_t stride, const ActView& a, float* y, int64_t n, int k, int batch) {
  const int upr = dev_units_per_row(QT, k);
  for (int64_t r = 0; r < n; ++r) {
    for (int b = 0; b < batch; ++b) {
      ActView ab{a.q + (int64_t)b * k, a.d + (int64_t)b * (k >> 5), a.s + (int64_t)b * (k >> 4), a.m + (int64_t)b * (k >> 6), k};
      // 32 lanes, each striding over units, then a tree reduction like the warp shuffle
      float lane[32];
      for (int l = 0; l < 32; ++l) { float acc = 0.f; for (int u = l; u < upr; u += 32) unit_dot<QT, 1>(W + r * stride, u, ab, &acc); lane[l] = acc; }
      for (int off = 16; off > 0; off >>= 1) for (int l = 0; l < off; ++l) lane[l] += lane[l + off];
      y[(int64_t)b * n + r] = lane[0];
    }
  }
}
}  // namespace

extern "C" {

int64_t rlz_dev_row_bytes(int qtype, int64_t k) { return dev_row_bytes(qtype, k); }

// y[batch, n] = W_dev[n, k] x[batch, k] with int8 activations, exactly as the GPU fast path computes it.
int rlz_emu_gemv(int qtype, const void* W, int64_t stride, const float* x, float* y, int64_t n, int k, int batch) {
  if (k % 32) return -1;
  std::vector<int8_t> q((size_t)batch * k); std::vector<float> d((size_t)batch * (k / 32));
  std::vector<int32_t> s((size_t)batch * (k / 16)); std::vector<U4> m((size_t)batch * (k / 64) + 1);
  for (int b = 0; b < batch; ++b)
    quantize_act_row(x + (int64_t)b * k, k, q.data() + (int64_t)b * k, d.data() + (int64_t)b * (k / 32), s.data() + (int64_t)b * (k / 16),
                     m.data() + (int64_t)b * (k / 64));
  ActView a{q.data(), d.data(), s.data(), m.data(), k};
  const uint8_t* w = (const uint8_t*)W;
  switch (qtype) {
    case QT_Q4_K: emu_rows<QT_Q4_K>(w, stride, a, y, n, k, batch); return 0;
    case QT_Q5_K: emu_rows<QT_Q5_K>(w, stride, a, y, n, k, batch); return 0;
    case QT_Q6_K: emu_rows<QT_Q6_K>(w, stride, a, y, n, k, batch); return 0;
    case QT_Q8_0: emu_rows<QT_Q8_0>(w, stride, a, y, n, k, batch); return 0;
    case QT_Q4_0: emu_rows<QT_Q4_0>(w, stride, a, y, n, k, batch); return 0;
    default: return -2;
  }
}


// Same product through the half-block functions of the streamed GEMV (csrc/gemv_blocks.h).
int rlz_emu_gemv_blocks(int qtype, const void* W, int64_t stride, const float* x, float* y, int64_t n, int k, int batch) {
  if (k % 256 || dev_block_bytes(qtype) == 0) return -1;
  std::vector<int8_t> q((size_t)batch * k); std::vector<U4> rec4((size_t)batch * (k / 64)); std::vector<F2> rec6((size_t)batch * (k / 16));
  for (int b = 0; b < batch; ++b)
    quantize_act_row_blk(x + (int64_t)b * k, k, q.data() + (int64_t)b * k, rec4.data() + (int64_t)b * (k / 64), rec6.data() + (int64_t)b * (k / 16));
  const int bb = dev_block_bytes(qtype), nsb = k / 256;
  for (int64_t r = 0; r < n; ++r)
    for (int b = 0; b < batch; ++b) {
      ActBlk ab{q.data() + (int64_t)b * k, rec4.data() + (int64_t)b * (k / 64), rec6.data() + (int64_t)b * (k / 16), k, nsb};
      float acc = 0.f;
      for (int sb = 0; sb < nsb; ++sb)
        for (int h = 0; h < 2; ++h) {
          const uint8_t* blk = (const uint8_t*)W + r * stride + (int64_t)sb * bb;
          float t = 0.f;
          if (qtype == QT_Q4_K) halfblock_dot<QT_Q4_K, 1>(blk, sb, h, ab, &t);
          else if (qtype == QT_Q5_K) halfblock_dot<QT_Q5_K, 1>(blk, sb, h, ab, &t);
          else halfblock_dot<QT_Q6_K, 1>(blk, sb, h, ab, &t);
          acc += t;
        }
      y[(int64_t)b * n + r] = acc;
    }
  return 0;
}

}  // extern "C"
