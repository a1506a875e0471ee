// Decode GEMV over block-quantised weights (batch 1..4), with the surrounding element-wise
// work fused in:
//   prologue : RMSNorm / LayerNorm of the input vector and its int8 quantisation (per CTA, in
//              shared memory) - no separate norm or quantise kernels, no activation round trip;
//   body     : one warp per output row, lanes stride over 16-byte weight units (dp4a);
//   epilogue : bias, GELU/SiLU, SwiGLU combine of a gate/up pair, second accumulated matrix
//              (parallel attention+MLP blocks), residual add.
// One launch covers up to four matrices that share the launch (e.g. Q, K, V or QKV + MLP-up).
//
// Replaces the reference's q4k/q5k/q6k/q8_0/q4_0 GEMV families, q8_quantize, the fused
// rmsnorm/gate-up/swiglu GEMVs, residual_add and bias kernels
// (src/cuda/executor/q4k_mwv_gemv.rs:7-945, src/cuda/executor/layers/gemv_dispatch.rs:53-309).
#include "common.cuh"
#include "../gemv_units.h"
#include "gemv_params.h"
#include "gemv_common.cuh"
#include "gemv_body.cuh"

namespace rlz {

template <int B, bool FAST>
__global__ void __launch_bounds__(GEMV_THREADS, (FAST && B <= GEMV_OCC2_MAXB ? 2 : 1)) gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  gemv_body<B, FAST, true>(p, (int)blockIdx.x, smem);
}

template <int B, bool FAST>
cudaError_t launch_gemv_t(const GemvParams& p, int grid, cudaStream_t stream) {
  const size_t smem = gemv_smem_bytes(p);
  static SmemOptIn opt;
  if (cudaError_t e = opt.ensure(gemv_kernel<B, FAST>, smem); e != cudaSuccess) return e;
  return launch(gemv_kernel<B, FAST>, dim3(grid), dim3(GEMV_THREADS), smem, stream, p);
}
template <int B>
cudaError_t launch_gemv(const GemvParams& p, int grid, cudaStream_t stream) {
  return p.any_generic ? launch_gemv_t<B, false>(p, grid, stream) : launch_gemv_t<B, true>(p, grid, stream);
}

}  // namespace rlz

extern "C" {

// Returns 0 on success, a negative value for invalid parameters, or a positive cudaError_t.
int rlz_gemv(const rlz::GemvParams* pp, void* stream) {
  using namespace rlz;
  GemvParams p = *pp;
  int grid = 0;
  const int rc = gemv_prepare(p, &grid);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  switch (p.batch) {
    case 1: e = launch_gemv<1>(p, grid, st); break;
    case 2: e = launch_gemv<2>(p, grid, st); break;
    case 3: e = launch_gemv<3>(p, grid, st); break;
    default: e = launch_gemv<4>(p, grid, st); break;
  }
  return (int)e;
}

// Diagnostics: phase trace of the one-launch-per-GEMV kernel (8 timestamps in ns per CTA: entry, dependency wait done,
// first input staged, first segment's rows done, second input staged, second segment's rows done, partial sums ready,
// epilogue done; unused points stay 0).
int rlz_gemv_trace_enable(int on) {
  const int v = on ? 1 : 0;
  return (int)cudaMemcpyToSymbol(rlz::g_gemv_trace_on, &v, sizeof(int));
}
int rlz_gemv_trace_read(unsigned long long* out, int ctas, int clear) {
  if (ctas < 1 || ctas > rlz::GEMV_TRACE_CTAS) return -1;
  cudaError_t e = cudaMemcpyFromSymbol(out, rlz::g_gemv_trace, sizeof(unsigned long long) * ctas * rlz::GEMV_TRACE_PTS);
  if (e != cudaSuccess || !clear) return (int)e;
  static unsigned long long zeros[rlz::GEMV_TRACE_CTAS * rlz::GEMV_TRACE_PTS];
  return (int)cudaMemcpyToSymbol(rlz::g_gemv_trace, zeros, sizeof(zeros));
}

// fills in the derived fields of *pp in place (for callers that embed the description in a step program)
int rlz_gemv_prepare(rlz::GemvParams* pp, int* grid_out) { return rlz::gemv_prepare(*pp, grid_out); }

// dynamic shared memory of a prepared launch description
long long rlz_gemv_smem_bytes(const rlz::GemvParams* pp) { return (long long)rlz::gemv_smem_bytes(*pp); }

int rlz_sizeof_gemv_params() { return (int)sizeof(rlz::GemvParams); }

}  // extern "C"
