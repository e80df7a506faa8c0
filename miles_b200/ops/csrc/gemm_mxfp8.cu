// Block-scaled MXFP8 GEMM on tcgen05:  C[M,N] (bf16) = (A ∘ 2^(sa−127)) · (B ∘ 2^(sb−127))ᵀ
//   A [M,K], B [N,K] e4m3 bytes (K-major);  sa [M, K/32], sb [N, K/32] e8m0 bytes: one scale per 1×32 block, the format
//   `mxfp8_quant` writes.  K must be a multiple of 128.
// The scaling happens inside the tensor core (`tcgen05.mma.kind::mxf8f6f4.block_scale`): each K=32 instruction multiplies
// its 32-element dot products by the row's and the column's scale before accumulating in fp32 TMEM, so no dequantised copy
// of either operand ever exists.  Pipeline per 128×128×128 stage:
//   warp 0   TMA: A and B tiles (128 rows × 128 bytes, 128-byte swizzle)
//   warps 6, 7  scale loaders (A and B): per row one 32-bit word = the 4 scales of this stage's 4 K blocks, written to shared
//            memory in the layout `tcgen05.cp.32x128b.warpx4` expects (row r = 32·m1 + m0 → byte 16·m0 + 4·m1 + kblock).  The
//            words of the NEXT four stages are already in flight (registers) while the current four are written: one lane's
//            loads touch 32 different rows, i.e. pure latency — with a single warp loading stage by stage the tensor pipe
//            idled 4/5 of the time (642 TFLOP/s, half the bf16 kernel)
//   warp 1   tcgen05.cp of both scale chunks into TMEM (4 columns each per 128 rows), then 4 MMAs with sf_id = 0..3
//   warps 2..5  epilogue (TMEM → bf16), accumulator double-buffered as in the bf16 GEMM
// Every wait is bounded; on a timeout the kernel raises the error flag, frees TMEM and returns.
#include "launch.h"
#include "ptx.cuh"

namespace mb {
namespace mx {

static constexpr int BM = 128, BN = 128, BK = 128;            // BK bytes = elements (fp8)
static constexpr int kStages = 5;
static constexpr int kABytes = BM * BK, kBBytes = BN * BK;    // 16 KB each
static constexpr int kSfBytes = 512;                          // 128 rows × 4 K blocks
static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
static constexpr int kBarOff = kStages * kStageBytes;
static constexpr int kSmemTotal = kBarOff + 256 + 4 * 4096 + 1024;   // + epilogue staging tiles
static constexpr uint32_t kTmemCols = 512;                    // 2 × 128 accumulator columns + 8 scale columns → next power of two
static constexpr uint32_t kSfaCol = 256, kSfbCol = 260;

struct Params {
  const uint8_t* sa;
  const uint8_t* sb;
  __nv_bfloat16* C;
  int M, N, K;
  long long ldc;
  int* error_flag;
  // grouped (MoE) form: rows of A are expert-sorted and padded to 128 per expert; tile_expert[m_blk] is the expert of each
  // row block (−1: a block past the rows in use — computed against expert 0 and not stored, so that every role of the CTA
  // walks the same tile sequence); B and its scales hold the experts stacked, N rows each.  null: one dense B.
  const int* tile_expert;
};

__device__ __forceinline__ int b_row_base(const Params& p, int m_blk) {
  if (p.tile_expert == nullptr) return 0;
  const int e = p.tile_expert[m_blk];
  return (e < 0 ? 0 : e) * p.N;
}

__global__ void __launch_bounds__(256, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOff);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_ptr + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_stages = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 3); mbar_init(&empty_bar[s], 1); }   // TMA thread + two scale warps
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

  auto stage_ptr = [&](int s) { return smem + s * kStageBytes; };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const int m_blk = t % m_tiles, n_blk = t / m_tiles;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 31); break; }
          mbar_expect_tx(&full_bar[stage], kABytes + kBBytes);
          tma_load_2d(stage_ptr(stage), &tmap_a, &full_bar[stage], ks * BK, m_blk * BM);
          tma_load_2d(stage_ptr(stage) + kABytes, &tmap_b, &full_bar[stage], ks * BK, b_row_base(p, m_blk) + n_blk * BN);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp >= 6) {
    // ---- scale loaders: warp 6 = A rows, warp 7 = B rows; lane = m0, four row groups m1; prefetch distance 4 stages ----
    const bool is_a = warp == 6;
    const int words_per_row = p.K / 128;                       // 32-bit words of 4 scales per row
    const uint32_t* src32 = reinterpret_cast<const uint32_t*>(is_a ? p.sa : p.sb);
    const int limit = is_a ? p.M : p.N;
    const long long n_items = static_cast<long long>((total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                                                     static_cast<int>(gridDim.x)) * k_stages;   // (tile, k stage) pairs of this CTA
    auto fetch = [&](long long item, uint32_t (&w)[4]) {
      if (item >= n_items) return;
      const int t = blockIdx.x + static_cast<int>(item / k_stages) * gridDim.x, ks = static_cast<int>(item % k_stages);
      const int blk = is_a ? t % m_tiles : t / m_tiles;
      const int base = is_a ? 0 : b_row_base(p, t % m_tiles);       // stacked experts: rows of this tile's expert
#pragma unroll
      for (int m1 = 0; m1 < 4; ++m1) {
        const int r = blk * 128 + m1 * 32 + lane;
        // rows past the matrix edge get scale 2^0: their operand rows are zero-filled, the products stay 0
        w[m1] = r < limit ? __ldg(src32 + static_cast<long long>(base + r) * words_per_row + ks) : 0x7f7f7f7fu;
      }
    };
    uint32_t cur[4][4], nxt[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) fetch(j, cur[j]);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (long long base = 0; base < n_items && ok && !*abort_flag; base += 4) {
#pragma unroll
      for (int j = 0; j < 4; ++j) fetch(base + 4 + j, nxt[j]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (base + j >= n_items) break;
        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
        uint32_t* sf = reinterpret_cast<uint32_t*>(stage_ptr(stage) + kABytes + kBBytes + (is_a ? 0 : kSfBytes));
#pragma unroll
        for (int m1 = 0; m1 < 4; ++m1) sf[lane * 4 + m1] = cur[j][m1];
        fence_proxy_async();                                    // generic-proxy writes → visible to tcgen05.cp
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int m1 = 0; m1 < 4; ++m1) cur[j][m1] = nxt[j][m1];
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.error_flag, 35); }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 32); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait(&full_bar[stage], phase)) { *abort_flag = 1; atomicExch(p.error_flag, 33); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(stage_ptr(stage));
          const uint32_t b_addr = a_addr + kABytes;
          const uint32_t sfa_addr = b_addr + kBBytes, sfb_addr = sfa_addr + kSfBytes;
          // scales of this stage → TMEM (4 columns each); ordered before the MMAs below in the tensor-core pipe
          tmem_cp_32x128b_warpx4(tmem_base + kSfaCol, make_smem_desc_noswizzle(sfa_addr, 128, 128));
          tmem_cp_32x128b_warpx4(tmem_base + kSfbCol, make_smem_desc_noswizzle(sfb_addr, 128, 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) {                          // 4 K blocks of 32 bytes inside the 128-byte swizzle row
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            const uint32_t sel = static_cast<uint32_t>(k) << 30;  // byte of the scale column, as in the idesc sf_id fields
            umma_mxf8(d_tmem, ad, bd, make_idesc_mxf8(BM, BN, k), (tmem_base + kSfaCol) | sel, (tmem_base + kSfbCol) | sel,
                      (ks | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp >= 2 && warp <= 5) {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      const int m_blk = t % m_tiles, n_blk = t / m_tiles;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.error_flag, 34); break; }
      tc_fence_after();
      const bool store = p.tile_expert == nullptr || p.tile_expert[m_blk] >= 0;
      const int row0 = m_blk * BM + q * 32;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      uint8_t* stage_tile = smem + kBarOff + 256 + q * 4096;
      const bool fast = ((reinterpret_cast<uintptr_t>(p.C) | (p.ldc * 2)) & 15) == 0 && (p.N & 7) == 0;
#pragma unroll 1
      for (int c2 = 0; c2 < BN / 64; ++c2) {
        const int colr = n_blk * BN + c2 * 64;
        if (colr >= p.N || !store) break;
        if (fast) {
          // 64 columns at a time through a 4 KB per-warp staging tile: every store instruction writes four full 128-byte lines
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
              *reinterpret_cast<uint4*>(stage_tile + lane * 128 + (((half * 4 + i) ^ (lane & 7)) << 4)) = o;
            }
          }
          __syncwarp();
          const int unit = lane & 7, col = colr + unit * 8;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rr = k * 4 + (lane >> 3);
            if (row0 + rr < p.M && col < p.N)
              *reinterpret_cast<uint4*>(p.C + static_cast<long long>(row0 + rr) * p.ldc + col) =
                  *reinterpret_cast<const uint4*>(stage_tile + rr * 128 + ((unit ^ (rr & 7)) << 4));
          }
          __syncwarp();
        } else {
          const int row = row0 + lane;
          for (int half = 0; half < 2; ++half) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c2 * 64 + half * 32, r);
            tmem_ld_wait();
            const int col0 = colr + half * 32;
            if (row < p.M)
              for (int i = 0; i < 32 && col0 + i < p.N; ++i)
                p.C[static_cast<long long>(row) * p.ldc + col0 + i] = __float2bfloat16(__uint_as_float(r[i]));
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

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_tmap_u8_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld_bytes) {
  static PFN_encodeTiled enc = nullptr;
  if (enc == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || ptr == nullptr)
      return -1;
    enc = reinterpret_cast<PFN_encodeTiled>(ptr);
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_bytes)};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    cudaFree(nullptr);
    r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace mx
}  // namespace mb

extern "C" int mb_gemm_mxfp8(const void* A, const void* sa, const void* B, const void* sb, void* C, int M, int N, int K, long long ldc,
                             int* error_flag, cudaStream_t stream) {
  using namespace mb::mx;
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 || K == 0) return -1;
  CUtensorMap ta, tb;
  int r = make_tmap_u8_2d(&ta, A, M, K, K);
  if (r) return 1000 + r;
  r = make_tmap_u8_2d(&tb, B, N, K, K);
  if (r) return 2000 + r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  Params p{static_cast<const uint8_t*>(sa), static_cast<const uint8_t*>(sb), static_cast<__nv_bfloat16*>(C), M, N, K, ldc, error_flag, nullptr};
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  gemm_mxfp8_kernel<<<tiles < sms ? tiles : sms, 256, kSmemTotal, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// Grouped (MoE) form.  A [M_pad, K] e4m3, expert-sorted rows padded to 128 per expert, sa its 1×32 scales; B [E·N, K] e4m3 with
// sb [E·N, K/32]; tile_expert [M_pad/128] (device) names the expert of every row block (−1: not in use, nothing stored);
// C [M_pad, N] bf16.  N must be a multiple of 128 so that a B tile never straddles two experts.
extern "C" int mb_gemm_mxfp8_grouped(const void* A, const void* sa, const void* B, const void* sb, void* C, int M_pad, int N, int K, int E,
                                     const int* tile_expert, long long ldc, int* error_flag, cudaStream_t stream) {
  using namespace mb::mx;
  if (M_pad <= 0 || N <= 0 || E <= 0) return 0;
  if (K % 128 || K == 0 || N % BN || M_pad % BM) return -1;
  CUtensorMap ta, tb;
  int r = make_tmap_u8_2d(&ta, A, M_pad, K, K);
  if (r) return 1000 + r;
  r = make_tmap_u8_2d(&tb, B, static_cast<long long>(E) * N, K, K);
  if (r) return 2000 + r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  Params p{static_cast<const uint8_t*>(sa), static_cast<const uint8_t*>(sb), static_cast<__nv_bfloat16*>(C), M_pad, N, K, ldc, error_flag,
           tile_expert};
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (M_pad / BM) * (N / BN);
  gemm_mxfp8_kernel<<<tiles < sms ? tiles : sms, 256, kSmemTotal, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}
