// Device-side primitives for kernels that talk to peer GPUs over NVLink through plain peer pointers:
// system-scope release/acquire flag signalling with time-bounded waits, and a small table of peer base addresses.
// No TMA or cluster multicast is used on peer memory anywhere: remote data moves with ordinary ld/st (16-byte vectors).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

static constexpr int kMaxRanks = 8;
static constexpr unsigned long long kPeerWaitLimitNs = 1000000000ull;  // 1 s, then give up and raise the error flag

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* addr) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Wait until *addr >= target (acquire).  Returns false after kPeerWaitLimitNs.
__device__ __forceinline__ bool wait_flag_ge(const int* addr, int target) {
  unsigned long long t0 = 0;
  for (unsigned i = 0;; ++i) {
    if (ld_acquire_sys(addr) >= target) return true;
    if ((i & 255u) == 255u) {
      const unsigned long long now = gtimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kPeerWaitLimitNs) return false;
    }
  }
}

// Flag layout on every rank: flags[channel * kMaxRanks + src_rank].
// One thread per peer publishes `epoch` into the peer's slot for this rank, then waits for every peer's epoch here.
// Must be called by at least `world` threads of ONE block after all of that block's prior global writes that peers
// will read are complete (a __syncthreads() + __threadfence_system() precede the store).  Returns false on timeout.
__device__ __forceinline__ bool cross_rank_barrier(const PeerPtrs& flags, int rank, int world, int channel, int epoch) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  __threadfence_system();
  if (static_cast<int>(threadIdx.x) < world) {
    int* remote = reinterpret_cast<int*>(flags.p[threadIdx.x]) + channel * kMaxRanks + rank;
    st_release_sys(remote, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + channel * kMaxRanks + threadIdx.x;
    if (!wait_flag_ge(mine, epoch)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}

}  // namespace mb
