// Device-side primitives for kernels that talk to peer GPUs over NVLink through plain peer pointers:
// system-scope release/acquire flag signalling with time-bounded waits, and a small table of peer base addresses.
// No TMA or cluster multicast is used on peer memory anywhere: remote data moves with ordinary ld/st (16-byte vectors).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

static constexpr int kMaxRanks = 8;
// How long a wait on a peer may poll before it gives up and raises the error flag, and where that flag lives.  Both are
// per translation unit (every .cu that includes this header has its own copy) and are set from the host with the unit's
// `*_configure` call; the default suits tests, production sets a few seconds (`Fabric.configure`).
static __device__ unsigned long long g_peer_wait_limit_ns = 2000000000ull;
static __device__ int* g_fabric_err = nullptr;

// True once any kernel of this process raised the error flag: kernels that would consume what a timed-out wait was
// guarding return at once instead (their outputs are then undefined; the host raises when it polls the flag).
__device__ __forceinline__ bool fabric_poisoned() {
  int* e = g_fabric_err;
  return e != nullptr && *reinterpret_cast<volatile int*>(e) != 0;
}

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

// Wait until *addr >= target (acquire).  Returns false after g_peer_wait_limit_ns.
__device__ __forceinline__ bool wait_flag_ge(const int* addr, int target) {
  unsigned long long t0 = 0;
  const unsigned long long limit = g_peer_wait_limit_ns;
  for (unsigned i = 0;; ++i) {
    if (ld_acquire_sys(addr) >= target) return true;
    if ((i & 255u) == 255u) {
      const unsigned long long now = gtimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit) return false;
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
    // a poisoned process still publishes its epoch (peers are not made to wait for it) but waits for nobody
    if (!fabric_poisoned() && !wait_flag_ge(mine, epoch)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}

// ---- split barrier: the producer kernel signals from its last block, the consumer kernel waits in its prologue -------------
// `publish_when_grid_done`: call with ALL threads of every block after the block's last global write that peers will read.
// The block that takes the last ticket advances the device-side epoch of `channel` and publishes it to every peer
// (release at system scope); `ticket` is one int that is zero between kernels (the last block resets it).
__device__ __forceinline__ void publish_when_grid_done(const PeerPtrs& flags, int rank, int world, int channel, int* epochs,
                                                       int* ticket) {
  __shared__ int last_sh, epoch_sh;
  // ONE thread per block fences at system scope, after the block barrier has ordered every thread's stores before it
  // (a system-scope fence from each of a block's 256 threads costs ~10 µs per kernel: measured)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int t = atomicAdd(ticket, 1);
    last_sh = (t == static_cast<int>(gridDim.x) - 1);
    if (last_sh) {
      __threadfence();                    // the other blocks' writes (ordered before their tickets) are visible here
      *ticket = 0;
      epoch_sh = ++epochs[channel];
      __threadfence_system();
    }
  }
  __syncthreads();
  if (last_sh && static_cast<int>(threadIdx.x) < world)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + channel * kMaxRanks + rank, epoch_sh);
}

// `wait_peers`: every block of the consumer waits (bounded) until all peers published the current epoch of `channel`.
// The epoch is read from device memory: the producer kernel of THIS rank advanced it earlier on the same stream.
__device__ __forceinline__ bool wait_peers(const PeerPtrs& flags, int rank, int world, int channel, const int* epochs) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world) {
    const int epoch = *reinterpret_cast<const volatile int*>(epochs + channel);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + channel * kMaxRanks + threadIdx.x;
    if (!fabric_poisoned() && !wait_flag_ge(mine, epoch)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}

// Host side of the two settings above for the including translation unit.
#define MB_DEFINE_FABRIC_CONFIGURE(fn_name)                                                                        \
  extern "C" int fn_name(int* err, unsigned long long wait_ns) {                                                  \
    cudaError_t e = cudaMemcpyToSymbol(mb::g_fabric_err, &err, sizeof(err));                                      \
    if (e != cudaSuccess) return static_cast<int>(e);                                                             \
    if (wait_ns) e = cudaMemcpyToSymbol(mb::g_peer_wait_limit_ns, &wait_ns, sizeof(wait_ns));                     \
    return static_cast<int>(e);                                                                                   \
  }

}  // namespace mb
