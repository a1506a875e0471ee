// Parameter block of the decode GEMV launch (mirrored field-for-field by ctypes structures
// in realizar_b200/ops/_signatures.py).
#pragma once
#include <stdint.h>

namespace rlz {

constexpr int GEMV_MAX_MATS = 4;
constexpr int GEMV_MAX_X = 4;

struct GemvSeg {            // one weight matrix contributing to the rows of a GemvMat
  const uint8_t* W;         // device layout, rows `stride` bytes apart
  int64_t stride;
  int32_t qtype;
  int32_t k;
  int32_t x_id;             // which input vector it multiplies
  int32_t _pad;
};

struct GemvMat {            // a block of output rows
  GemvSeg seg[2];
  const float* bias;        // added to segment 0 (or to the sum when combine == ADD)
  const float* bias2;       // added to segment 1 (gated combine) or to the sum
  int32_t nseg;             // 1 or 2
  int32_t combine;          // COMBINE_* for two segments
  int32_t n;                // rows
  int32_t out_off;          // column offset in y
  int32_t act;              // ACT_* applied after combine/bias
  int32_t has_residual;     // add p.residual[b, row]
  int32_t rows_per_cta;
  int32_t cta_begin;        // filled by the launcher
};

struct GemvX {              // an input vector (batch rows `ld` floats apart) and its fused norm
  const float* x;
  const float* nw;          // norm weight (may be null)
  const float* nb;          // norm bias (may be null)
  int64_t ld;
  int32_t k;
  int32_t norm;             // NORM_*
  float eps;
  int32_t _pad;
};

struct GemvParams {
  GemvMat mat[GEMV_MAX_MATS];
  GemvX xs[GEMV_MAX_X];
  float* y;
  const float* residual;
  int64_t ldy;
  int64_t ld_res;
  int32_t nmat;
  int32_t batch;
  int32_t max_k;            // filled by the launcher
  int32_t max_rows;         // filled by the launcher
  int32_t any_generic;      // filled by the launcher
  int32_t _pad;
};

}  // namespace rlz
