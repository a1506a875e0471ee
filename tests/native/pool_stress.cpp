// Stress of the host library's thread pool and batched products, built with -fsanitize=thread by tests/test_sanitizers.py:
// several caller threads issue parallel products at once (the pool serialises them), results must be the same every time.
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
int rlz_matvec(int qtype, const void* W, const float* x, float* y, int64_t n, int64_t k, int64_t batch);
int rlz_quantize(int qtype, const float* src, void* dst, int64_t n, int64_t k);
int64_t rlz_row_bytes(int qtype, int64_t k);
void rlz_parallel_for(int64_t n, int64_t chunk, void (*fn)(int64_t, int64_t, void*), void* ctx);
}

static void bump(int64_t a, int64_t b, void* ctx) { ((std::atomic<int64_t>*)ctx)->fetch_add(b - a); }

int main() {
  const int QT_Q4_K = 12, QT_Q8_0 = 8;
  const int64_t n = 96, k = 512;
  std::vector<float> w((size_t)n * k), x((size_t)5 * k);
  uint32_t s = 12345;
  auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.f - 1.f; };
  for (auto& v : w) v = rnd();
  for (auto& v : x) v = rnd();
  int bad = 0;
  for (int qt : {QT_Q4_K, QT_Q8_0}) {
    std::vector<uint8_t> q((size_t)n * rlz_row_bytes(qt, k));
    if (rlz_quantize(qt, w.data(), q.data(), n, k)) { std::printf("quantize failed\n"); return 2; }
    std::vector<float> ref((size_t)5 * n);
    rlz_matvec(qt, q.data(), x.data(), ref.data(), n, k, 5);
    std::vector<std::thread> callers;
    std::atomic<int> mism{0};
    for (int t = 0; t < 3; ++t)
      callers.emplace_back([&] {
        std::vector<float> y((size_t)5 * n);
        for (int it = 0; it < 60; ++it) {
          rlz_matvec(qt, q.data(), x.data(), y.data(), n, k, 5);
          if (std::memcmp(y.data(), ref.data(), y.size() * sizeof(float))) mism.fetch_add(1);
          std::atomic<int64_t> total{0};
          rlz_parallel_for(1000, 7, bump, &total);
          if (total.load() != 1000) mism.fetch_add(1);
        }
      });
    for (auto& c : callers) c.join();
    bad += mism.load();
  }
  std::printf("POOL-STRESS %s\n", bad ? "MISMATCH" : "OK");
  return bad ? 3 : 0;
}
