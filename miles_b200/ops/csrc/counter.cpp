// Process-wide count of kernel-launcher calls made by this extension (reported by the benchmark as `gpu_launches`).
#include <atomic>

static std::atomic<long long> g_launches{0};

extern "C" void mb_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long mb_launch_count() { return g_launches.load(std::memory_order_relaxed); }
