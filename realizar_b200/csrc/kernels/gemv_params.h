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
  // batch 1 only: besides the fp32 store, write the outputs as the int8 activation of the NEXT launch (the layout that
  // launch stages in shared memory: codes, per-64 records, per-32 scales, per-16 sums), so that it copies instead of quantising
  uint8_t* q_out;           // destination activation block (null = off); rows_per_cta and q_out_col0 are multiples of 32
  int32_t q_out_k;          // length of the destination activation vector
  int32_t q_out_col0;       // column of output row 0 in that vector
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
  const uint8_t* pre;       // batch 1: this input already quantised by the producing launch (see GemvMat::q_out), or null
};

constexpr int GEMV_AR_MAX_RANKS = 8;

// In-kernel all-reduce of the outputs of a row-parallel GEMV over peer memory (tensor parallel).
// Low-latency protocol without fences or separate flags: every value travels as one 8-byte store
// {float bits, step epoch}.  A rank stores its partial rows into slot [parity][rank] of every
// rank's inbox; each output element is then polled (bounded) in every slot until its epoch word
// matches, and the values are summed in rank order.  parity = epoch & 1 keeps a slot from being
// overwritten while a slower rank still reads the previous step.
// Inbox of one call site: [parity 2][rank][4 batch rows][n] pairs of 32-bit words.
struct GemvAr {
  uint2* inbox[GEMV_AR_MAX_RANKS];        // rank r's inbox for this call site (own entry = local memory)
  const uint32_t* epoch;                  // device word, incremented once per step before the first use
  int32_t* status;                        // device word receiving an error code when a wait expires
  int64_t spin_limit;                     // polls per element before giving up
  int32_t rank, world, enabled, n;        // n = elements per batch row in the inbox
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
  GemvAr ar;                // all-reduce of matrix 0's outputs (single-matrix launches only)
};

}  // namespace rlz
