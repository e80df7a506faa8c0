// Device-side index checks of the DEBUG build of the extension (-DMILES_DEBUG_BOUNDS, `python -m miles_b200.ops.build --debug`).
//
// Kernels that take indices from tensors (cache slots, block-table entries, token rows) call in_bounds(which, index, code)
// before using one.  In the normal build the call is `true` and costs nothing.  In the debug build it compares the index
// with a limit the host published for that kind of index; an index outside [0, limit) is RECORDED (how many, and the first
// one's code / value / limit) and the access is SKIPPED — the kernel never traps and never touches the bad address, so the
// context stays usable and the host can read what went wrong (`bounds_report()` in the Python module).
// One record and one limit table per translation unit (no relocatable device code needed).
#pragma once
#include <cuda_runtime.h>

namespace mb {
namespace dbg {

enum Limit { kKvSlots = 0, kMoePairs = 1, kKvBlocks = 2, kNumLimits = 4 };

#ifdef MILES_DEBUG_BOUNDS
static __device__ long long g_limit[kNumLimits] = {-1, -1, -1, -1};   // −1: not published, not checked
static __device__ unsigned long long g_record[4];                      // count, first code, first index, its limit

__device__ __forceinline__ bool in_bounds(int which, long long idx, int code) {
  const long long lim = g_limit[which];
  if (lim < 0 || (idx >= 0 && idx < lim)) return true;
  if (atomicAdd(&g_record[0], 1ull) == 0ull) {
    g_record[1] = static_cast<unsigned long long>(code);
    g_record[2] = static_cast<unsigned long long>(idx);
    g_record[3] = static_cast<unsigned long long>(lim);
  }
  return false;
}
#else
__device__ __forceinline__ bool in_bounds(int, long long, int) { return true; }
#endif

}  // namespace dbg
}  // namespace mb

// Host API of a translation unit: <prefix>_set_limit(which, value) publishes a limit (−1 switches the check off),
// <prefix>_read(out4, clear) copies {count, code, index, limit} out.  Both return −1 in a build without the checks.
#ifdef MILES_DEBUG_BOUNDS
#define MB_DEFINE_BOUNDS_API(prefix)                                                                                       \
  extern "C" int prefix##_set_limit(int which, long long value) {                                                           \
    if (which < 0 || which >= mb::dbg::kNumLimits) return -2;                                                               \
    return static_cast<int>(cudaMemcpyToSymbol(mb::dbg::g_limit, &value, sizeof(value), which * sizeof(long long)));        \
  }                                                                                                                         \
  extern "C" int prefix##_read(long long* out4, int clear) {                                                                \
    unsigned long long r[4];                                                                                                \
    cudaError_t e = cudaMemcpyFromSymbol(r, mb::dbg::g_record, sizeof(r));                                                  \
    if (e != cudaSuccess) return static_cast<int>(e);                                                                       \
    for (int i = 0; i < 4; ++i) out4[i] = static_cast<long long>(r[i]);                                                     \
    if (clear) {                                                                                                            \
      const unsigned long long z[4] = {0, 0, 0, 0};                                                                         \
      e = cudaMemcpyToSymbol(mb::dbg::g_record, z, sizeof(z));                                                              \
    }                                                                                                                       \
    return static_cast<int>(e);                                                                                             \
  }
#else
#define MB_DEFINE_BOUNDS_API(prefix)                                      \
  extern "C" int prefix##_set_limit(int, long long) { return -1; }        \
  extern "C" int prefix##_read(long long*, int) { return -1; }
#endif
