// Library-wide runtime state: launch counter, programmatic-dependent-launch switch,
// device queries and small utilities exported to Python.
#include "common.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>

namespace rlz {
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_pdl{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
}  // namespace rlz

extern "C" {

long long rlz_launch_count() { return rlz::g_launches.load(); }
void rlz_launch_count_reset() { rlz::g_launches.store(0); }
void rlz_set_pdl(int on) { rlz::g_pdl.store(on ? 1 : 0); }
int rlz_get_pdl() { return rlz::g_pdl.load(); }

// compute capability (major*10+minor) and SM count of a device, or a negative cudaError_t
int rlz_device_info(int device, int* sm_count, long long* total_mem) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return -(int)e;
  if (sm_count) *sm_count = prop.multiProcessorCount;
  if (total_mem) *total_mem = (long long)prop.totalGlobalMem;
  return prop.major * 10 + prop.minor;
}

const char* rlz_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
int rlz_cuda_last_error() { return (int)cudaGetLastError(); }

}  // extern "C"
