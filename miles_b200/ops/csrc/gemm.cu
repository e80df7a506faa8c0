// bf16 GEMM on the 5th-generation tensor cores: TMA → shared memory (128-byte swizzle) → tcgen05.mma with the
// fp32 accumulator in tensor memory → tcgen05.ld epilogue.  Persistent, warp-specialised:
//   warp 0       TMA producer (one elected lane)
//   warp 1       TMEM allocation + MMA issue (one elected lane)
//   warps 2..5   epilogue: each owns the TMEM lane quadrant (warp_idx % 4), i.e. 32 rows of the 128-row tile
// The accumulator is double buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
//
// One kernel template covers
//   C[M,N] = A · Bᵀ with A and B each either K-major ([rows, K] row-major) or MN-major ([K, rows] row-major):
//     forward  y = x·Wᵀ      A = x  [M,K]  K-major     B = W  [N,K]  K-major
//     dgrad    dx = dy·W     A = dy [M,N'] K-major     B = W  [N',K'] as [K=N', N=K'] MN-major
//     wgrad    dW = dyᵀ·x    A = dy [T,N'] MN-major    B = x  [T,K'] MN-major   (reduction over tokens)
//   grouped forward/dgrad (MoE): rows of A are expert-sorted and padded to 128 per expert; `tile_expert[m_blk]`
//     selects which expert's weight block B uses (−1 = unused tile).
//   grouped wgrad: one output [N',K'] per expert, reduction over that expert's row segment.
// Every mbarrier wait is bounded; on timeout the kernel raises `*error_flag`, drains and frees TMEM, and returns.
#include "ptx.cuh"
#include "launch.h"
#include "pdl.cuh"

namespace mb {

static constexpr int BM = 128;
static constexpr int BK = 64;       // 64 bf16 = 128 bytes = one swizzle row
static constexpr int UMMA_K = 16;

enum GemmMode { kDense = 0, kGroupedFwd = 1, kGroupedWgrad = 2 };

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;           // elements
  long long group_stride_c;  // elements between per-group outputs (grouped wgrad)
  int out_fp32;
  int accumulate;
  const __nv_bfloat16* bias;
  const int* tile_expert;  // grouped fwd: [m_tiles]
  const int* seg_offsets;  // grouped wgrad: [groups+1], multiples of BK
  int num_groups;
  int b_group_rows;        // grouped fwd: rows of B per expert (N for K-major B, K for MN-major B)
  int* error_flag;
  // split-K (dense, few output tiles): `split_k` CTAs share one output tile, each writing the partial sums of its K slice
  // to its own fp32 plane of `ws` [split_k, M, N]; the last to arrive (counter per tile and 32-row quadrant) adds the
  // planes in slice order, writes C and resets the counter
  int split_k;
  float* ws;
  int* counters;
};

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStagingBytes = 4 * 4096;   // epilogue: one 32-row × 128-byte transposition tile per warp
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + kStagingBytes + 1024;  // + alignment slack
};

template <int BN, int A_MN, int B_MN, int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * L::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;        // [2]
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_ptr + 1);
  uint8_t* smem_stage = smem + kStages * L::kStageBytes + L::kBarrierBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tiles_per_group = m_tiles * n_tiles;
  const int split_k = (MODE == kDense && p.split_k > 1) ? p.split_k : 1;
  // "group" = expert (grouped wgrad) or K slice (dense split-K): both index the outer tile dimension
  const int total_tiles = (MODE == kGroupedWgrad) ? tiles_per_group * p.num_groups : tiles_per_group * split_k;
  constexpr bool kOuter = (MODE == kGroupedWgrad || MODE == kDense);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  // everything above (barrier init, TMEM allocation, descriptor prefetch) may overlap the tail of the previous kernel
  pdl_trigger();
  pdl_wait();

  auto k_range = [&](int group, int& k0, int& k_blocks) {
    if (MODE == kGroupedWgrad) {
      k0 = p.seg_offsets[group];
      k_blocks = (p.seg_offsets[group + 1] - k0) / BK;
    } else {
      const int total_kb = (p.K + BK - 1) / BK;
      const int per = (total_kb + split_k - 1) / split_k;
      const int lo = group * per;                       // group = K slice (0 without split-K)
      k0 = lo * BK;
      k_blocks = max(0, min(per, total_kb - lo));
    }
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const int group = kOuter ? t / tiles_per_group : 0;
        const int tt = kOuter ? t % tiles_per_group : t;
        const int m_blk = tt % m_tiles, n_blk = tt / m_tiles;
        int b_row_off = 0;
        if (MODE == kGroupedFwd) {
          const int e = p.tile_expert[m_blk];
          if (e < 0) continue;
          b_row_off = e * p.b_group_rows;
        }
        int k0, k_blocks;
        k_range(group, k0, k_blocks);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 1); break; }
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          const int kc = k0 + kb * BK;
          uint8_t* sa = smem_a + stage * L::kABytes;
          uint8_t* sb = smem_b + stage * L::kBBytes;
          if (A_MN) {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d(sa + a * (BK * 128), &tmap_a, &full_bar[stage], m_blk * BM + a * 64, kc);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kc, m_blk * BM);
          }
          if (B_MN) {
            // MN-major B for grouped fwd stacks experts along K rows: [E·K, N]
#pragma unroll
            for (int a = 0; a < BN / 64; ++a)
              tma_load_2d(sb + a * (BK * 128), &tmap_b, &full_bar[stage], n_blk * BN + a * 64, kc + b_row_off);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kc, n_blk * BN + b_row_off);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const int group = kOuter ? t / tiles_per_group : 0;
        const int tt = kOuter ? t % tiles_per_group : t;
        const int m_blk = tt % m_tiles;
        if (MODE == kGroupedFwd && p.tile_expert[m_blk] < 0) continue;
        int k0, k_blocks;
        k_range(group, k0, k_blocks);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 2); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { *abort_flag = 1; atomicExch(p.error_flag, 3); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * L::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * L::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);   // frees the smem stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (k_blocks == 0) {
          // empty reduction range (an expert without tokens): the epilogue writes zeros, nothing to wait for
        }
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      const int group = kOuter ? t / tiles_per_group : 0;
      const int tt = kOuter ? t % tiles_per_group : t;
      const int m_blk = tt % m_tiles, n_blk = tt / m_tiles;
      if (MODE == kGroupedFwd && p.tile_expert[m_blk] < 0) continue;
      int k0, k_blocks;
      k_range(group, k0, k_blocks);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.error_flag, 4); break; }
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (MODE == kDense && split_k > 1) {
        // ---- split-K: add this slice's partial sums to the workspace; the last slice to arrive finishes the tile ----
        // ws holds one [M, N] fp32 plane per K slice: plain vector stores, no atomics
        float* wrow = p.ws + (static_cast<long long>(group) * p.M + row) * p.N;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col0 = n_blk * BN + c * 32;
          if (row < p.M && col0 < p.N) {
            if (k_blocks == 0) {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                __stcg(reinterpret_cast<float4*>(wrow + col0 + i),
                       make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                   __uint_as_float(r[i + 3])));
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) __stcg(wrow + col0 + i, __uint_as_float(r[i]));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        // one counter per (tile, 32-row quadrant): the rows a warp reduced are finished by the last warp to arrive for
        // that quadrant, so no CTA-wide barrier is needed (and none can be left waiting on an error path)
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = (atomicAdd(&p.counters[tt * 4 + q], 1) == split_k - 1) ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          const int row_lo = m_blk * BM + q * 32;
          const int col_hi = min(p.N, (n_blk + 1) * BN);
          const long long plane_sz = static_cast<long long>(p.M) * p.N;
          if (BN == 64 && ((p.N | p.ldc) & 3) == 0 && (n_blk + 1) * BN <= p.N && p.bias == nullptr && !p.accumulate) {
            // fast path: 16 lanes × float4 cover the 64 columns of a row, two rows per instruction, 4 row pairs and
            // 4 planes in flight at once (the loop is latency-bound otherwise)
            const int half = lane >> 4, c = n_blk * BN + (lane & 15) * 4;
#pragma unroll 1
            for (int i0 = 0; i0 < 16 && row_lo + 2 * i0 < p.M; i0 += 4) {
              float4 acc[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
              for (int s = 0; s < split_k; ++s) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int rr = row_lo + 2 * (i0 + j) + half;
                  if (rr < p.M) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(p.ws + s * plane_sz + static_cast<long long>(rr) * p.N + c));
                    acc[j].x += v.x; acc[j].y += v.y; acc[j].z += v.z; acc[j].w += v.w;
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int rr = row_lo + 2 * (i0 + j) + half;
                if (rr >= p.M) continue;
                if (p.out_fp32) {
                  *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + static_cast<long long>(rr) * p.ldc + c) = acc[j];
                } else {
                  uint2 o;
                  o.x = pack_bf16x2(acc[j].x, acc[j].y);
                  o.y = pack_bf16x2(acc[j].z, acc[j].w);
                  *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(rr) * p.ldc + c) = o;
                }
              }
            }
          } else
          for (int rr = row_lo; rr < min(p.M, row_lo + 32); ++rr) {      // lanes sweep the columns of one row: coalesced
            const float* w = p.ws + static_cast<long long>(rr) * p.N;
            const long long plane = static_cast<long long>(p.M) * p.N;
            uint8_t* c_row = reinterpret_cast<uint8_t*>(p.C) + static_cast<long long>(rr) * p.ldc * (p.out_fp32 ? 4 : 2);
            for (int col = n_blk * BN + lane; col < col_hi; col += 32) {
              float v = 0.f;
              for (int s = 0; s < split_k; ++s) v += __ldcg(w + s * plane + col);   // fixed order: deterministic
              if (p.bias != nullptr) v += __bfloat162float(p.bias[col]);
              if (p.out_fp32) {
                float* d = reinterpret_cast<float*>(c_row) + col;
                *d = p.accumulate ? *d + v : v;
              } else {
                reinterpret_cast<__nv_bfloat16*>(c_row)[col] = __float2bfloat16(v);
              }
            }
          }
          __syncwarp();
          if (lane == 0) p.counters[tt * 4 + q] = 0;
        }
        continue;
      }
      // Coalesced path: the accumulator arrives one row per thread, but whole 128-byte lines are what the memory system
      // wants.  Each warp turns 128 bytes of output per row at a time (64 bf16 or 32 fp32 columns) through its staging tile
      // (16-byte units, XOR-swizzled against bank conflicts): written row-per-lane, read back with 8 lanes covering one
      // row, so every store instruction writes four full lines.  Needs 16-byte aligned rows; otherwise the plain path below.
      const int esz = p.out_fp32 ? 4 : 2;
      const int cols_per_round = 128 / esz;
      if ((((p.ldc * esz) | (p.group_stride_c * esz) | static_cast<long long>(reinterpret_cast<uintptr_t>(p.C))) & 15) == 0 &&
          (p.N * esz) % 16 == 0) {
        const int row0 = m_blk * BM + q * 32;
        uint8_t* stage = smem_stage + q * 4096;
        uint8_t* c_tile = reinterpret_cast<uint8_t*>(p.C) +
                          (static_cast<long long>(group) * p.group_stride_c + static_cast<long long>(row0) * p.ldc) * esz;
#pragma unroll 1
        for (int c2 = 0; c2 < BN / cols_per_round; ++c2) {
          const int colr = n_blk * BN + c2 * cols_per_round;
          if (colr >= p.N) break;                                  // uniform over the warp
          if (p.out_fp32) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c2 * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 o;
              o.x = (k_blocks == 0) ? 0.f : __uint_as_float(r[4 * i]);
              o.y = (k_blocks == 0) ? 0.f : __uint_as_float(r[4 * i + 1]);
              o.z = (k_blocks == 0) ? 0.f : __uint_as_float(r[4 * i + 2]);
              o.w = (k_blocks == 0) ? 0.f : __uint_as_float(r[4 * i + 3]);
              *reinterpret_cast<float4*>(stage + lane * 128 + ((i ^ (lane & 7)) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t r[32];
              tmem_ld_32x32(t_row + c2 * 64 + half * 32, r);
              tmem_ld_wait();
              if (k_blocks == 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
              }
              if (p.bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const int col = colr + half * 32 + i;
                  if (col < p.N) r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(p.bias[col]));
                }
              }
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
          }
          __syncwarp();
          const int unit = lane & 7;
          const int col = colr + unit * (16 / esz);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rr = k * 4 + (lane >> 3);
            if (row0 + rr < p.M && col < p.N) {
              uint8_t* dst = c_tile + (static_cast<long long>(rr) * p.ldc + col) * esz;
              if (p.out_fp32) {
                float4 o = *reinterpret_cast<const float4*>(stage + rr * 128 + ((unit ^ (rr & 7)) << 4));
                if (p.bias != nullptr) {
                  o.x += __bfloat162float(p.bias[col]); o.y += __bfloat162float(p.bias[col + 1]);
                  o.z += __bfloat162float(p.bias[col + 2]); o.w += __bfloat162float(p.bias[col + 3]);
                }
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = o;
              } else {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((unit ^ (rr & 7)) << 4));
              }
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) +
                        (static_cast<long long>(group) * p.group_stride_c + static_cast<long long>(row) * p.ldc) *
                            (p.out_fp32 ? 4 : 2);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = (k_blocks == 0) ? 0.f : __uint_as_float(r[i]);
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
          }
          const bool full = (col0 + 32 <= p.N);
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(c_base) + col0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + i) = o;
              }
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_base) + col0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                o.x = pack_bf16x2(v[i], v[i + 1]);
                o.y = pack_bf16x2(v[i + 2], v[i + 3]);
                o.z = pack_bf16x2(v[i + 4], v[i + 5]);
                o.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = __float2bfloat16(v[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess || ptr == nullptr) return nullptr;
    fn = reinterpret_cast<PFN_encodeTiled>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension `ld` (elements);
// box = [box_rows, box_cols] with 128-byte swizzle (box_cols·2 bytes must be 128).
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows,
                      int box_cols) {
  PFN_encodeTiled enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a host thread that has not made a runtime call yet (e.g. an autograd worker) has no context bound:
    // bind the device's primary context and encode again
    cudaFree(nullptr);
    r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, int A_MN, int B_MN, int MODE>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int total_tiles, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = total_tiles < num_sms() ? total_tiles : num_sms();
  if (grid <= 0) return 0;
  return static_cast<int>(launch_pdl(kern, dim3(grid), dim3(192), L::kTotal, stream, ta, tb, p));
}

template <int A_MN, int B_MN, int MODE>
static int launch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int tiles, cudaStream_t s) {
  switch (bn) {
    case 256: return launch_one<256, A_MN, B_MN, MODE>(ta, tb, p, tiles, s);
    case 128: return launch_one<128, A_MN, B_MN, MODE>(ta, tb, p, tiles, s);
    default: return launch_one<64, A_MN, B_MN, MODE>(ta, tb, p, tiles, s);
  }
}

static int pick_bn(int M, int N, int forced) {
  if (forced == 256 || forced == 128 || forced == 64) return forced;
  // largest tile width that still gives every SM a tile
  const int sms = num_sms();
  const int m_tiles = (M + BM - 1) / BM;
  if (m_tiles * ((N + 255) / 256) >= sms) return 256;
  if (m_tiles * ((N + 127) / 128) >= sms) return 128;
  return 64;
}

}  // namespace mb

using namespace mb;

// C[M,N] = op(A)·op(B)ᵀ.  a_mn / b_mn: operand stored [K, rows] (MN-major) instead of [rows, K].
// lda / ldb are the leading dimensions (elements) of the stored matrices.
extern "C" int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate, const void* bias,
                            int force_bn, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int bn = pick_bn(M, N, force_bn);
  CUtensorMap ta, tb;
  int r;
  r = a_mn ? make_tmap_bf16_2d(&ta, A, K, M, lda, BK, 64) : make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
  if (r) return 1000 + r;
  r = b_mn ? make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, 64) : make_tmap_bf16_2d(&tb, B, N, K, ldb, bn, BK);
  if (r) return 2000 + r;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.error_flag = error_flag;
  p.num_groups = 1;
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  if (!a_mn && !b_mn) return launch_bn<0, 0, kDense>(bn, ta, tb, p, tiles, stream);
  if (!a_mn && b_mn) return launch_bn<0, 1, kDense>(bn, ta, tb, p, tiles, stream);
  if (a_mn && b_mn) return launch_bn<1, 1, kDense>(bn, ta, tb, p, tiles, stream);
  return launch_bn<1, 0, kDense>(bn, ta, tb, p, tiles, stream);
}

// Split-K form of C[M,N] = A[M,K]·B[N,K]ᵀ for decode-sized problems (few output tiles, long K): `split_k` CTAs per
// 128×64 tile each stream a K slice, so a GEMM with 32 output tiles still pulls weights with 128 SMs.
// ws: fp32 [split_k, M, N] workspace (contents irrelevant), counters: int [4 · tiles], zero on entry and zero again on exit.
extern "C" int mb_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                   long long ldc, int out_fp32, int accumulate, const void* bias, int split_k, float* ws,
                                   int* counters, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (split_k < 1 || ws == nullptr || counters == nullptr) return -1;
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
  if (r) return 1000 + r;
  r = make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK);
  if (r) return 2000 + r;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.error_flag = error_flag;
  p.num_groups = 1;
  p.split_k = split_k; p.ws = ws; p.counters = counters;
  const int tiles = ((M + BM - 1) / BM) * ((N + 63) / 64) * split_k;
  return launch_one<64, 0, 0, kDense>(ta, tb, p, tiles, stream);
}

// Grouped forward / dgrad: A [M_pad, K] expert-sorted rows (each expert's segment padded to 128 rows),
// tile_expert[M_pad/128] = expert of each row block (−1 → skip).  B holds all experts stacked:
//   b_mn = 0: B [E·N, K] (forward: W13 [E,2F,H] → N=2F,K=H;  W2 [E,H,F] → N=H,K=F)
//   b_mn = 1: B [E·K, N] (dgrad through the same weights: dX = dY·W uses W [E, K=rows, N=cols])
extern "C" int mb_gemm_bf16_grouped(const void* A, const void* B, void* C, int M_pad, int N, int K, int num_experts,
                                    const int* tile_expert, int b_mn, int out_fp32, int force_bn, int* error_flag,
                                    cudaStream_t stream) {
  if (M_pad <= 0 || N <= 0) return 0;
  const int bn = pick_bn(M_pad, N, force_bn);
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, A, M_pad, K, K, BM, BK);
  if (r) return 1000 + r;
  r = b_mn ? make_tmap_bf16_2d(&tb, B, static_cast<long long>(num_experts) * K, N, N, BK, 64)
           : make_tmap_bf16_2d(&tb, B, static_cast<long long>(num_experts) * N, K, K, bn, BK);
  if (r) return 2000 + r;
  GemmParams p{};
  p.M = M_pad; p.N = N; p.K = K; p.C = C; p.ldc = N; p.out_fp32 = out_fp32;
  p.tile_expert = tile_expert;
  p.b_group_rows = b_mn ? K : N;
  p.error_flag = error_flag;
  p.num_groups = num_experts;
  const int tiles = (M_pad / BM) * ((N + bn - 1) / bn);
  if (b_mn) return launch_bn<0, 1, kGroupedFwd>(bn, ta, tb, p, tiles, stream);
  return launch_bn<0, 0, kGroupedFwd>(bn, ta, tb, p, tiles, stream);
}

// Grouped wgrad: dW[e] [N, K] (+)= dY[seg_e, N]ᵀ · X[seg_e, K]; seg_offsets[E+1] are row offsets (multiples of 128).
extern "C" int mb_gemm_bf16_grouped_wgrad(const void* dY, const void* X, void* dW, int M_pad, int N, int K,
                                          int num_experts, const int* seg_offsets, int out_fp32, int accumulate,
                                          int force_bn, int* error_flag, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || num_experts <= 0) return 0;
  const int bn = pick_bn(N * num_experts, K, force_bn);
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, dY, M_pad, N, N, BK, 64);   // MN-major A: [tokens (k), N (m)]
  if (r) return 1000 + r;
  r = make_tmap_bf16_2d(&tb, X, M_pad, K, K, BK, 64);        // MN-major B: [tokens (k), K (n)]
  if (r) return 2000 + r;
  GemmParams p{};
  p.M = N; p.N = K; p.K = 0; p.C = dW; p.ldc = K; p.group_stride_c = static_cast<long long>(N) * K;
  p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.seg_offsets = seg_offsets;
  p.num_groups = num_experts;
  p.error_flag = error_flag;
  const int tiles = ((N + BM - 1) / BM) * ((K + bn - 1) / bn) * num_experts;
  return launch_bn<1, 1, kGroupedWgrad>(bn, ta, tb, p, tiles, stream);
}
