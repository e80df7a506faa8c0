// Tensor-parallel GEMMs fused with their sequence-parallel collective, one kernel each (tcgen05 + TMA + NVLink peers):
//
//  all-gather → GEMM   y[T, N] = gather_r(x_r[T/w, K]) · Wᵀ.  The A operand has one tensor map per rank over that rank's
//      staged x (peer memory for r ≠ rank).  Tiles are visited owner by owner starting with this rank, the TMA producer
//      waits (bounded) for the owner's "staged" flag the first time it needs that owner, then loads the tile straight from
//      the peer's memory into shared memory — no gathered copy of x is ever written.  (Plain TMA loads, no multicast.)
//
//  GEMM → reduce-scatter   out[T/w, N] = Σ_r (x_r[T, K/w] · W_rᵀ)[rows of this rank].  Every rank writes its partial tiles
//      into its own symmetric buffer, visiting destination row blocks starting with the *next* rank so that the blocks
//      other ranks wait for are finished first; when the last tile of a destination is stored the epilogue publishes a
//      flag to that rank.  After its tiles each CTA joins the reduction of this rank's row block, reading the partial
//      rows of every peer with 16-byte loads once their flags have arrived.
//
// Pipeline and warp roles are those of gemm.cu (warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, double-buffered TMEM).
#include "comm.cuh"
#include "launch.h"
#include "ptx.cuh"

namespace mb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows, int box_cols);

static constexpr int CBM = 128, CBK = 64, CUMMA_K = 16;
enum CommMode { kAllGather = 0, kReduceScatter = 1 };

struct TmapArray {
  CUtensorMap m[kMaxRanks];
};

struct CommGemmParams {
  int M, N, K;
  void* C;              // AG: y [M, N];  RS: this rank's partial buffer [M, N]
  long long ldc;
  int rank, world, rows_per_rank;
  PeerPtrs flags;
  int channel, epoch;
  PeerPtrs partials;    // RS: every rank's partial buffer
  void* out;            // RS: [rows_per_rank, N]
  int* dest_counters;   // RS: [world], zero on entry
  int* error_flag;
};

template <int BN>
struct CSmem {
  static constexpr int kABytes = CBM * CBK * 2;
  static constexpr int kBBytes = BN * CBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN >= 256) ? 4 : 6;
  static constexpr int kTotal = kStages * kStageBytes + 256 + 1024;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_comm_kernel(const __grid_constant__ TmapArray tmaps_a, const __grid_constant__ CUtensorMap tmap_b, CommGemmParams p) {
  using L = CSmem<BN>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = (2 * BN <= 256) ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * L::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mb_per_rank = p.rows_per_rank / CBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tiles_per_owner = mb_per_rank * n_tiles;
  const int total_tiles = tiles_per_owner * p.world;
  const int k_blocks = (p.K + CBK - 1) / CBK;
  int* my_flags = reinterpret_cast<int*>(p.flags.p[p.rank]) + p.channel * kMaxRanks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (MODE == kAllGather && blockIdx.x == 0 && warp == 2 && lane < p.world) {
    // tell every peer that this rank's staged x (written by the preceding kernel on this stream) is ready
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(p.flags.p[lane]) + p.channel * kMaxRanks + p.rank, p.epoch);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  // tile t → (owner/destination rank, m block, n block); own blocks first for AG, last for RS
  auto decode = [&](int t, int& owner, int& m_blk, int& n_blk) {
    const int i = t / tiles_per_owner, rem = t % tiles_per_owner;
    owner = (MODE == kAllGather) ? (p.rank + i) % p.world : (p.rank + 1 + i) % p.world;
    m_blk = owner * mb_per_rank + rem % mb_per_rank;
    n_blk = rem / mb_per_rank;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int ready_owner = p.rank;   // owners are visited in order; each needs one flag wait
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        int owner, m_blk, n_blk;
        decode(t, owner, m_blk, n_blk);
        if (MODE == kAllGather && owner != p.rank && owner != ready_owner) {
          if (!wait_flag_ge(my_flags + owner, p.epoch)) { *abort_flag = 1; atomicExch(p.error_flag, 11); break; }
          fence_proxy_async();
          ready_owner = owner;
        }
        const CUtensorMap* ta = (MODE == kAllGather) ? &tmaps_a.m[owner] : &tmaps_a.m[0];
        const int a_row = (MODE == kAllGather) ? (m_blk - owner * mb_per_rank) * CBM : m_blk * CBM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 12); break; }
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(smem_a + stage * L::kABytes, ta, &full_bar[stage], kb * CBK, a_row);
          tma_load_2d(smem_b + stage * L::kBBytes, &tmap_b, &full_bar[stage], kb * CBK, n_blk * BN);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(CBM, BN, 0, 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 13); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { *abort_flag = 1; atomicExch(p.error_flag, 14); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * L::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * L::kBBytes);
#pragma unroll
          for (int k = 0; k < CBK / CUMMA_K; ++k) {
            umma_bf16(d_tmem, make_smem_desc_sw128(a_addr + k * (CUMMA_K * 2), 16, 1024),
                      make_smem_desc_sw128(b_addr + k * (CUMMA_K * 2), 16, 1024), idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;
    const int etid = threadIdx.x - 64;   // 0..127 within the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      int owner, m_blk, n_blk;
      decode(t, owner, m_blk, n_blk);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.error_flag, 15); break; }
      tc_fence_after();
      const int row = m_blk * CBM + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* dst = c_row + col0;
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
              *reinterpret_cast<uint4*>(dst + i) = o;
            }
          } else {
            for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (MODE == kReduceScatter) {
        // publish "all partial tiles for `owner` are stored" once the last of them is done
        epi_bar_sync();
        if (etid == 0) {
          __threadfence_system();
          const int old = atomicAdd(&p.dest_counters[owner], 1);
          if (old == tiles_per_owner - 1)
            st_release_sys(reinterpret_cast<int*>(p.flags.p[owner]) + p.channel * kMaxRanks + p.rank, p.epoch);
        }
      }
    }
    if (MODE == kReduceScatter && !*abort_flag) {
      // reduction of this rank's row block out of every rank's partial buffer
      bool ok = true;
      for (int r = 0; r < p.world && ok; ++r) ok = wait_flag_ge(my_flags + r, p.epoch);
      if (!ok) {
        atomicExch(p.error_flag, 16);
      } else {
        const long long nvec = static_cast<long long>(p.rows_per_rank) * p.N / 8;
        const long long base = static_cast<long long>(p.rank) * p.rows_per_rank * p.N / 8;
        for (long long v = blockIdx.x * 128ll + etid; v < nvec; v += static_cast<long long>(gridDim.x) * 128) {
          float accv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int r = 0; r < p.world; ++r) {
            const uint4 raw = reinterpret_cast<const uint4*>(p.partials.p[r])[base + v];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(h[i]);
              accv[2 * i] += f.x;
              accv[2 * i + 1] += f.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(accv[0], accv[1]);
          o.y = pack_bf16x2(accv[2], accv[3]);
          o.z = pack_bf16x2(accv[4], accv[5]);
          o.w = pack_bf16x2(accv[6], accv[7]);
          reinterpret_cast<uint4*>(p.out)[v] = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, int MODE>
static int launch_comm(const TmapArray& ta, const CUtensorMap& tb, const CommGemmParams& p, int tiles, cudaStream_t s) {
  using L = CSmem<BN>;
  auto kern = gemm_comm_kernel<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 192, L::kTotal, s>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mb

using namespace mb;

// x_ptrs[r]: rank r's staged x [rows_per_rank, K] (bf16, row-major) as mapped in this process.
extern "C" int mb_ag_gemm(const long long* x_ptrs, const void* W, void* Y, int rows_per_rank, int N, int K, int rank, int world,
                          const long long* flag_ptrs, int channel, int epoch, int* error_flag, cudaStream_t s) {
  if (world > kMaxRanks || rows_per_rank % CBM || K % 8) return -1;
  TmapArray ta;
  for (int r = 0; r < world; ++r) {
    const int rc = make_tmap_bf16_2d(&ta.m[r], reinterpret_cast<const void*>(x_ptrs[r]), rows_per_rank, K, K, CBM, CBK);
    if (rc) return 1000 + rc;
  }
  for (int r = world; r < kMaxRanks; ++r) ta.m[r] = ta.m[0];
  const int M = rows_per_rank * world;
  const int bn = ((M / CBM) * ((N + 255) / 256) >= sm_count()) ? 256 : 128;
  CUtensorMap tb;
  int rc = make_tmap_bf16_2d(&tb, W, N, K, K, bn, CBK);
  if (rc) return 2000 + rc;
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = Y; p.ldc = N; p.rank = rank; p.world = world; p.rows_per_rank = rows_per_rank;
  for (int r = 0; r < kMaxRanks; ++r) p.flags.p[r] = (r < world) ? reinterpret_cast<void*>(flag_ptrs[r]) : nullptr;
  p.channel = channel; p.epoch = epoch; p.error_flag = error_flag;
  const int tiles = (M / CBM) * ((N + bn - 1) / bn);
  return bn == 256 ? launch_comm<256, kAllGather>(ta, tb, p, tiles, s) : launch_comm<128, kAllGather>(ta, tb, p, tiles, s);
}

// X [T, K] local; W [N, K]; partial_ptrs[r]: rank r's partial buffer [T, N] bf16; out [T/world, N]; counters [world] ints.
extern "C" int mb_gemm_rs(const void* X, const void* W, const long long* partial_ptrs, void* out, int* counters, int T, int N, int K,
                          int rank, int world, const long long* flag_ptrs, int channel, int epoch, int* error_flag, cudaStream_t s) {
  if (world > kMaxRanks || T % (CBM * world) || K % 8 || N % 8) return -1;
  const int rows_per_rank = T / world;
  TmapArray ta;
  int rc = make_tmap_bf16_2d(&ta.m[0], X, T, K, K, CBM, CBK);
  if (rc) return 1000 + rc;
  for (int r = 1; r < kMaxRanks; ++r) ta.m[r] = ta.m[0];
  const int bn = ((T / CBM) * ((N + 255) / 256) >= sm_count()) ? 256 : 128;
  CUtensorMap tb;
  rc = make_tmap_bf16_2d(&tb, W, N, K, K, bn, CBK);
  if (rc) return 2000 + rc;
  cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(int) * world, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  CommGemmParams p{};
  p.M = T; p.N = N; p.K = K; p.C = reinterpret_cast<void*>(partial_ptrs[rank]); p.ldc = N; p.rank = rank; p.world = world;
  p.rows_per_rank = rows_per_rank;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.flags.p[r] = (r < world) ? reinterpret_cast<void*>(flag_ptrs[r]) : nullptr;
    p.partials.p[r] = (r < world) ? reinterpret_cast<void*>(partial_ptrs[r]) : nullptr;
  }
  p.channel = channel; p.epoch = epoch; p.out = out; p.dest_counters = counters; p.error_flag = error_flag;
  const int tiles = (T / CBM) * ((N + bn - 1) / bn);
  return bn == 256 ? launch_comm<256, kReduceScatter>(ta, tb, p, tiles, s) : launch_comm<128, kReduceScatter>(ta, tb, p, tiles, s);
}
