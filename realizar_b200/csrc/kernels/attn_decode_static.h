// Allocation-free entry point for the flash-decode attention kernel.
//
// This entry point has no counterpart in the reference implementation.
//
// Who it is for: callers that are not allowed to allocate device memory at the point where they
// need attention - for example code running inside a memory-budgeted serving process whose pool
// has been handed out completely, a plugin loaded into a host application that owns the CUDA
// allocator, or a latency-critical loop that must not touch cudaMalloc (which synchronises the
// device).  The regular entry point, rlz_attn_decode, needs two scratch buffers from the caller
// (split-K partial results and per-head arrival counters); this variant keeps that scratch in a
// fixed array that lives inside the library image, so the caller passes inputs and outputs only.
//
// Limits (checked on every call; a launch that does not fit is rejected with
// RLZ_STATIC_TOO_LARGE and nothing is launched):
//   batch * n_heads * splits * (head_dim + 2)  <= RLZ_ATTN_STATIC_MAX_PARTIAL_FLOATS
//   batch * n_heads                            <= RLZ_ATTN_STATIC_MAX_COUNTERS
// The arrays take (RLZ_ATTN_STATIC_MAX_PARTIAL_FLOATS + RLZ_ATTN_STATIC_MAX_COUNTERS) * 4 bytes
// (about 4.1 MB) on every GPU that loads the library, until the process exits.
//
// Behaviour to know about:
//   * The first call on each device looks up the device address of the arrays and clears the
//     counters.  Make that first call on a device before starting any stream capture on it.
//   * The entry point itself calls no cudaMalloc / cudaFree or any other allocating routine.
//   * All calls on a device share the one scratch area, and it keeps whatever the previous call
//     left in it.  The kernel resets every counter it used before it finishes, so back-to-back
//     calls on one stream are safe; two calls that may run at the same time on the GPU (different
//     streams, or different host threads without ordering) race on the scratch and must not be made.
//   * `partial` and `counters` in the parameter block are ignored.
#pragma once
#include <stdint.h>

#define RLZ_ATTN_STATIC_MAX_PARTIAL_FLOATS (1 << 20)
#define RLZ_ATTN_STATIC_MAX_COUNTERS (1 << 14)
#define RLZ_STATIC_TOO_LARGE (-10)
#define RLZ_STATIC_NO_DEVICE (-11)

#ifdef __cplusplus
namespace rlz { struct AttnDecodeParams; }
extern "C" {
// Same arguments and return convention as rlz_attn_decode (0 = launched, > 0 = cudaError_t,
// < 0 = rejected).  `stream` is a cudaStream_t.
int rlz_attn_decode_static(const rlz::AttnDecodeParams* params, void* stream);
// Human-readable text for the negative codes above; never null.
const char* rlz_attn_decode_static_strerror(int code);
}
#endif
