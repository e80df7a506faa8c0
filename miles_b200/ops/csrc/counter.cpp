// Process-wide count of kernel-launcher calls made by this extension (reported by the benchmark as `gpu_launches`), and the
// switch for programmatic dependent launch (see pdl.cuh).
#include <atomic>
#include <cstdlib>
#include <cstring>

static std::atomic<long long> g_launches{0};
static std::atomic<int> g_pdl{-1};

extern "C" void mb_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long mb_launch_count() { return g_launches.load(std::memory_order_relaxed); }

// 1 = kernels that support it are launched with the programmatic-stream-serialization attribute (default; MILES_PDL=0 disables)
extern "C" int mb_pdl_enabled() {
  int v = g_pdl.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = std::getenv("MILES_PDL");
    v = (e != nullptr && std::strcmp(e, "0") == 0) ? 0 : 1;
    g_pdl.store(v, std::memory_order_relaxed);
  }
  return v;
}
extern "C" void mb_set_pdl(int on) { g_pdl.store(on ? 1 : 0, std::memory_order_relaxed); }
