// Tensor-parallel GEMMs fused with their sequence-parallel collective, one kernel each (tcgen05 + TMA + NVLink peers):
//
//  all-gather → GEMM   y[T, N] = gather_r(x_r[T/w, K]) · Wᵀ.  Every rank keeps a symmetric [T, K] buffer whose own row
//      block holds its x.  Four copy warps per CTA bring each remote row block over NVLink ONCE into the same rows of the
//      local buffer (16-byte peer loads, several in flight per thread) after the owner's "staged" flag arrived, and count
//      finished pieces per 128-row block; the TMA producer visits this rank's blocks first, waits (bounded) for a remote
//      block's count, then loads its tiles from LOCAL memory for every N tile.  The remote bytes cross NVLink once, not
//      once per N tile, and later tiles hit this GPU's L2.  (Plain TMA loads from local memory, no multicast.)
//
//  GEMM → reduce-scatter   out[T/w, N] = Σ_r (x_r[T, K/w] · W_rᵀ)[rows of this rank].  Every rank owns a symmetric buffer
//      of `world` slots [T/w, N]; the epilogue PUSHES each finished partial tile straight into slot `rank` of the
//      destination rank's buffer (peer stores from the registers that hold the tile), visiting destinations starting with
//      the next rank; when the last tile for a destination is stored a flag is published to it.  After its tiles each
//      CTA joins the reduction of this rank's row block, now a sum over LOCAL slots.  No full [T, N] partial is written
//      locally and nothing is pulled.
//
// Pipeline and warp roles are those of gemm.cu (warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, double-buffered TMEM);
// warps 6-9 exist only in the all-gather kernel (the copy warps).
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
  void* C;              // AG: y [M, N]
  long long ldc;
  int rank, world, rows_per_rank;
  PeerPtrs flags;
  int channel, epoch;
  PeerPtrs partials;    // RS: every rank's slot buffer [world, rows_per_rank, N];  AG: every rank's gathered buffer [M, K]
  void* out;            // RS: [rows_per_rank, N]
  int* dest_counters;   // RS: [world], zero on entry;  AG: [M / 128] pieces copied per row block, zero on entry
  int* error_flag;
};

template <int BN>
struct CSmem {
  static constexpr int kABytes = CBM * CBK * 2;
  static constexpr int kBBytes = BN * CBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN >= 256) ? 4 : 6;
  static constexpr int kTotal = kStages * kStageBytes + 256 + 4 * 4096 + 1024;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void copy_bar_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
static constexpr int kCopyPieces = 8;        // a 128-row block is copied in 8 pieces of 16 rows
static constexpr int kCopyThreads = 128;

template <int BN, int MODE>
__global__ void __launch_bounds__(MODE == kAllGather ? 320 : 192, 1)
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
  volatile int* copy_go = abort_flag + 1;     // the copy warps' shared decision for the current piece
  uint8_t* smem_stage = smem + kStages * L::kStageBytes + 256;   // 4 epilogue warps × 4 KB

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
      int ready_blk = -1;         // a CTA meets the tiles of one row block consecutively (m fastest): one wait per block
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        int owner, m_blk, n_blk;
        decode(t, owner, m_blk, n_blk);
        if (MODE == kAllGather && owner != p.rank && m_blk != ready_blk) {
          // the copy warps of the whole grid bring this block in; wait until all its pieces are in local memory
          const unsigned long long limit = g_peer_wait_limit_ns + kWaitLimitNs;
          unsigned long long t0 = 0;
          bool ok = true;
          for (unsigned i = 0; ld_acquire_gpu(p.dest_counters + m_blk) < kCopyPieces; ++i) {
            if ((i & 255u) == 255u) {
              const unsigned long long now = gtimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > limit || *abort_flag) { ok = false; break; }
            }
          }
          if (!ok) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 11); break; }
          fence_proxy_async_all();
          ready_blk = m_blk;
        }
        const CUtensorMap* ta = &tmaps_a.m[0];
        const int a_row = m_blk * CBM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 12); break; }
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
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 13); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 14); ok = false; break; }
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
  } else if (MODE == kAllGather && warp >= 6) {
    // copy warps: remote row blocks → the same rows of the local gathered buffer, owner by owner in the order the tiles
    // need them; pieces are dealt round-robin over the grid so that every block is finished by many CTAs at once
    const int ctid = threadIdx.x - 192;
    const long long row_vecs = p.K / 8;                                  // 16-byte vectors per row
    const long long piece_vecs = (CBM / kCopyPieces) * row_vecs;
    uint4* local = reinterpret_cast<uint4*>(p.partials.p[p.rank]);
    const int pieces_per_owner = mb_per_rank * kCopyPieces;
    const int total_pieces = pieces_per_owner * (p.world - 1);
    int ready_owner = -1;
    for (int pc = blockIdx.x; pc < total_pieces; pc += gridDim.x) {
      const int owner = (p.rank + 1 + pc / pieces_per_owner) % p.world;
      const int rem = pc % pieces_per_owner;
      const int m_blk = owner * mb_per_rank + rem / kCopyPieces;
      // one thread decides for all 128 (waits for the owner's flag when a new owner starts); the others learn it behind a
      // barrier, so that no thread can leave the loop while another still heads for a barrier
      if (ctid == 0) {
        bool go = !*abort_flag;
        if (go && owner != ready_owner && !wait_flag_ge(my_flags + owner, p.epoch)) {
          *abort_flag = 1;
          atomicCAS(p.error_flag, 0, 17);
          go = false;
        }
        *copy_go = go ? 1 : 0;
      }
      ready_owner = owner;
      copy_bar_sync();
      if (!*copy_go) break;
      const long long base = (static_cast<long long>(m_blk) * kCopyPieces + rem % kCopyPieces) * piece_vecs;
      const uint4* src = reinterpret_cast<const uint4*>(p.partials.p[owner]) + base;
      uint4* dst = local + base;
      long long v = ctid;
      for (; v + 7 * kCopyThreads < piece_vecs; v += 8 * kCopyThreads) {
        uint4 r[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) r[u] = ld_peer16(src + v + u * kCopyThreads);
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[v + u * kCopyThreads] = r[u];
      }
      for (; v < piece_vecs; v += kCopyThreads) dst[v] = ld_peer16(src + v);
      fence_proxy_async_all();
      __threadfence();
      copy_bar_sync();
      if (ctid == 0) atomicAdd(p.dest_counters + m_blk, 1);
    }
  } else {
    const int q = warp & 3;
    const int etid = threadIdx.x - 64;   // 0..127 within the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      int owner, m_blk, n_blk;
      decode(t, owner, m_blk, n_blk);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 15); break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      // The accumulator arrives one ROW per thread; global (and above all peer) stores want whole 128-byte lines.  Each warp
      // turns 64 columns at a time through its 4 KB staging tile (16-byte units, XOR-swizzled against bank conflicts):
      // written row-per-lane, read back with 8 lanes covering one row's 128 bytes, so that every store instruction
      // writes four full lines.
      const int row0 = m_blk * CBM + q * 32;                      // first row of this warp's 32
      uint8_t* stage = smem_stage + q * 4096;
      // RS: the tile goes into slot `rank` of the destination's buffer (peer memory unless owner == rank)
      __nv_bfloat16* c_base = (MODE == kAllGather)
          ? reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row0) * p.ldc
          : reinterpret_cast<__nv_bfloat16*>(p.partials.p[owner]) +
                (static_cast<long long>(p.rank) * p.rows_per_rank + (row0 - owner * p.rows_per_rank)) * p.ldc;
#pragma unroll 1
      for (int c2 = 0; c2 < BN / 64; ++c2) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c2 * 64 + half * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
            *reinterpret_cast<uint4*>(stage + lane * 128 + (((half * 4 + i) ^ (lane & 7)) << 4)) = o;
          }
        }
        __syncwarp();
        const int unit = lane & 7;
        const int col = n_blk * BN + c2 * 64 + unit * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int rr = k * 4 + (lane >> 3);
          const uint4 o = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((unit ^ (rr & 7)) << 4));
          if (row0 + rr < p.M && col < p.N) *reinterpret_cast<uint4*>(c_base + static_cast<long long>(rr) * p.ldc + col) = o;
        }
        __syncwarp();
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
        atomicCAS(p.error_flag, 0, 16);
      } else {
        const long long nvec = static_cast<long long>(p.rows_per_rank) * p.N / 8;
        const uint4* slots = reinterpret_cast<const uint4*>(p.partials.p[p.rank]);
        for (long long v = blockIdx.x * 128ll + etid; v < nvec; v += static_cast<long long>(gridDim.x) * 128) {
          float accv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int r = 0; r < p.world; ++r) {
            const uint4 raw = slots[r * nvec + v];
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
  kern<<<grid, MODE == kAllGather ? 320 : 192, L::kTotal, s>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mb

using namespace mb;

MB_DEFINE_FABRIC_CONFIGURE(mb_gemm_comm_configure)

// xg_ptrs[r]: rank r's symmetric gathered buffer [rows_per_rank·world, K] (bf16, row-major) as mapped in this process;
// rank r has written its own x into rows [r·rows_per_rank, (r+1)·rows_per_rank) of its buffer before this launch.
// block_counters: [rows_per_rank·world / 128] ints (zeroed here).
extern "C" int mb_ag_gemm(const long long* xg_ptrs, const void* W, void* Y, int* block_counters, int rows_per_rank, int N, int K,
                          int rank, int world, const long long* flag_ptrs, int channel, int epoch, int* error_flag, cudaStream_t s) {
  if (world > kMaxRanks || rows_per_rank % CBM || K % 8 || N % 8) return -1;
  const int M = rows_per_rank * world;
  TmapArray ta;
  const int rc0 = make_tmap_bf16_2d(&ta.m[0], reinterpret_cast<const void*>(xg_ptrs[rank]), M, K, K, CBM, CBK);   // LOCAL memory only
  if (rc0) return 1000 + rc0;
  for (int r = 1; r < kMaxRanks; ++r) ta.m[r] = ta.m[0];
  const int bn = ((M / CBM) * ((N + 255) / 256) >= sm_count()) ? 256 : 128;
  CUtensorMap tb;
  int rc = make_tmap_bf16_2d(&tb, W, N, K, K, bn, CBK);
  if (rc) return 2000 + rc;
  cudaError_t e = cudaMemsetAsync(block_counters, 0, sizeof(int) * (M / CBM), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = Y; p.ldc = N; p.rank = rank; p.world = world; p.rows_per_rank = rows_per_rank;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.flags.p[r] = (r < world) ? reinterpret_cast<void*>(flag_ptrs[r]) : nullptr;
    p.partials.p[r] = (r < world) ? reinterpret_cast<void*>(xg_ptrs[r]) : nullptr;
  }
  p.channel = channel; p.epoch = epoch; p.error_flag = error_flag; p.dest_counters = block_counters;
  const int tiles = (M / CBM) * ((N + bn - 1) / bn);
  return bn == 256 ? launch_comm<256, kAllGather>(ta, tb, p, tiles, s) : launch_comm<128, kAllGather>(ta, tb, p, tiles, s);
}

// X [T, K] local; W [N, K]; partial_ptrs[r]: rank r's slot buffer [world, T/world, N] bf16; out [T/world, N]; counters [world] ints.
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
  p.M = T; p.N = N; p.K = K; p.C = nullptr; p.ldc = N; p.rank = rank; p.world = world;
  p.rows_per_rank = rows_per_rank;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.flags.p[r] = (r < world) ? reinterpret_cast<void*>(flag_ptrs[r]) : nullptr;
    p.partials.p[r] = (r < world) ? reinterpret_cast<void*>(partial_ptrs[r]) : nullptr;
  }
  p.channel = channel; p.epoch = epoch; p.out = out; p.dest_counters = counters; p.error_flag = error_flag;
  const int tiles = (T / CBM) * ((N + bn - 1) / bn);
  return bn == 256 ? launch_comm<256, kReduceScatter>(ta, tb, p, tiles, s) : launch_comm<128, kReduceScatter>(ta, tb, p, tiles, s);
}
