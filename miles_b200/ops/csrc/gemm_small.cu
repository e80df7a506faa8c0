// Operand-swapped GEMM for decode-sized token counts:  C[tokens, N] = X[tokens, K] · W[N, K]ᵀ  with tokens ≤ a few hundred.
//
// The general kernel (gemm.cu) puts tokens on the 128-row M side of the MMA: with 1…64 tokens two thirds of every pipeline
// stage are padding rows and a projection exposes only N/64 CTAs.  Here the WEIGHT rows are the M side (128 output features
// per tile, every byte loaded is a weight byte that must be read anyway) and the tokens are the N side in tiles of
// BT ∈ {16, 32, 64}; the accumulator D[feature, token] is written back transposed.  Parallelism comes from split-K
// (dense: K slices → fp32 planes, last arriver reduces) or from the experts (grouped).
//   dense    tiles = ⌈N/128⌉ × ⌈tokens/BT⌉ × split_k
//   grouped  X = expert-sorted rows whose segments are padded to BT (`moe_align` with pad = BT), tile_expert[token tile] gives
//            the expert (−1: unused tile); W = [E·N, K] stacked.  tiles = ⌈N/128⌉ × token tiles
// Same pipeline as gemm.cu: warp 0 TMA, warp 1 tcgen05.mma (TMEM accumulator ×2), warps 2–5 epilogue; bounded waits.
#include "launch.h"
#include "pdl.cuh"
#include "ptx.cuh"

namespace mb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows, int box_cols);

namespace sm {

static constexpr int BMW = 128;     // weight rows (output features) per tile
static constexpr int BK = 64;
static constexpr int kStages = 8;

struct Params {
  int tokens, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  const __nv_bfloat16* bias;
  const int* tile_expert;      // grouped: [token tiles]
  const int* used_rows;        // grouped: device count of rows in use (a multiple of the token tile); tiles beyond it are not visited
  int grouped;
  int split_k;
  float* ws;                   // [split_k, tokens, N]
  int* counters;               // [4 · output tiles]
  int* error_flag;
};

template <int BT>
struct Layout {
  static constexpr int kABytes = BMW * BK * 2;         // weights: 16 KB
  static constexpr int kBBytes = BT * BK * 2;          // tokens: 2 / 4 / 8 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTotal = kStages * kStageBytes + 256 + 1024;
};

template <int BT>
__global__ void __launch_bounds__(192, 1)
gemm_small_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, Params p) {
  using L = Layout<BT>;
  constexpr uint32_t kTmemCols = (2 * BT < 32) ? 32 : 2 * BT;
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  pdl_trigger();
  pdl_wait();

  const int n_tiles = (p.N + BMW - 1) / BMW;
  // `used_rows` is written by a preceding kernel of the stream: read it only after the dependency wait
  int t_tiles = (p.tokens + BT - 1) / BT;
  if (p.grouped && p.used_rows != nullptr) t_tiles = min(t_tiles, (*p.used_rows + BT - 1) / BT);
  const int out_tiles = n_tiles * t_tiles;
  const int split_k = p.split_k > 1 ? p.split_k : 1;
  const int total = out_tiles * split_k;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb_per = (total_kb + split_k - 1) / split_k;

  // tile id → (feature tile, token tile, K slice); consecutive CTAs take different feature tiles of the same tokens
  auto decode = [&](int t, int& n_blk, int& t_blk, int& slice) {
    slice = t / out_tiles;
    const int o = t % out_tiles;
    n_blk = o % n_tiles;
    t_blk = o / n_tiles;
  };
  auto k_range = [&](int slice, int& kb0, int& kbs) {
    kb0 = slice * kb_per;
    kbs = max(0, min(kb_per, total_kb - kb0));
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
        int n_blk, t_blk, slice, kb0, kbs;
        decode(t, n_blk, t_blk, slice);
        int w_row = n_blk * BMW;
        if (p.grouped) {
          const int e = p.tile_expert[t_blk];
          if (e < 0) continue;
          w_row += e * p.N;
        }
        k_range(slice, kb0, kbs);
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 41); break; }
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          const int kc = (kb0 + kb) * BK;
          tma_load_2d(smem_a + stage * L::kABytes, &tmap_w, &full_bar[stage], kc, w_row);
          tma_load_2d(smem_b + stage * L::kBBytes, &tmap_x, &full_bar[stage], kc, t_blk * BT);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BMW, BT, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
        int n_blk, t_blk, slice, kb0, kbs;
        decode(t, n_blk, t_blk, slice);
        if (p.grouped && p.tile_expert[t_blk] < 0) continue;
        k_range(slice, kb0, kbs);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 42); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BT;
        bool ok = true;
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { *abort_flag = 1; atomicExch(p.error_flag, 43); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * L::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * L::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 16, 1024), make_smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc,
                      (kb | k) != 0);
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
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
      int n_blk, t_blk, slice, kb0, kbs;
      decode(t, n_blk, t_blk, slice);
      if (p.grouped && p.tile_expert[t_blk] < 0) continue;
      k_range(slice, kb0, kbs);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.error_flag, 44); break; }
      tc_fence_after();
      const int n = n_blk * BMW + q * 32 + lane;                 // output feature of this thread
      const int tok0 = t_blk * BT;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BT;
      float v[BT];
#pragma unroll
      for (int c = 0; c < BT / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x16(t_row + c * 16, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) v[c * 16 + i] = kbs > 0 ? __uint_as_float(r[i]) : 0.f;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);              // the accumulator is in registers now
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      const bool n_ok = n < p.N;
      if (split_k == 1) {
        const float b = (p.bias != nullptr && n_ok) ? __bfloat162float(p.bias[n]) : 0.f;
        if (n_ok) {
#pragma unroll
          for (int i = 0; i < BT; ++i) {
            const int tok = tok0 + i;
            if (tok >= p.tokens) break;
            // lanes hold consecutive features: each token row gets one coalesced 64-byte (bf16) store per warp
            if (p.out_fp32) reinterpret_cast<float*>(p.C)[static_cast<long long>(tok) * p.ldc + n] = v[i] + b;
            else reinterpret_cast<__nv_bfloat16*>(p.C)[static_cast<long long>(tok) * p.ldc + n] = __float2bfloat16(v[i] + b);
          }
        }
        continue;
      }
      // ---- split-K: this slice's plane, then the last arriver of (tile, quadrant) adds the planes in slice order ----
      if (n_ok) {
        float* plane = p.ws + static_cast<long long>(slice) * p.tokens * p.N;
#pragma unroll
        for (int i = 0; i < BT; ++i) {
          const int tok = tok0 + i;
          if (tok >= p.tokens) break;
          __stcg(plane + static_cast<long long>(tok) * p.N + n, v[i]);
        }
      }
      __threadfence();
      __syncwarp();
      const int o = t % out_tiles;
      int last = 0;
      if (lane == 0) last = (atomicAdd(&p.counters[o * 4 + q], 1) == split_k - 1) ? 1 : 0;
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence();
        if (n_ok) {
          const float b = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
          const long long plane_sz = static_cast<long long>(p.tokens) * p.N;
          // one slice at a time with all BT loads of the slice in flight (the loads of a token are independent)
#pragma unroll
          for (int i = 0; i < BT; ++i) v[i] = b;
          for (int sl = 0; sl < split_k; ++sl) {
            const float* src = p.ws + sl * plane_sz + static_cast<long long>(tok0) * p.N + n;
#pragma unroll
            for (int i = 0; i < BT; ++i)
              if (tok0 + i < p.tokens) v[i] += __ldcg(src + static_cast<long long>(i) * p.N);
          }
#pragma unroll
          for (int i = 0; i < BT; ++i) {
            const int tok = tok0 + i;
            if (tok >= p.tokens) break;
            if (p.out_fp32) reinterpret_cast<float*>(p.C)[static_cast<long long>(tok) * p.ldc + n] = v[i];
            else reinterpret_cast<__nv_bfloat16*>(p.C)[static_cast<long long>(tok) * p.ldc + n] = __float2bfloat16(v[i]);
          }
        }
        __syncwarp();
        if (lane == 0) p.counters[o * 4 + q] = 0;
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

template <int BT>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, const Params& p, int tiles, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_small_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<BT>::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = tiles < sms ? tiles : sms;
  if (grid <= 0) return 0;
  return static_cast<int>(launch_pdl(gemm_small_kernel<BT>, dim3(grid), dim3(192), Layout<BT>::kTotal, s, tw, tx, p));
}

static int dispatch(int bt, const CUtensorMap& tw, const CUtensorMap& tx, const Params& p, int tiles, cudaStream_t s) {
  switch (bt) {
    case 16: return launch<16>(tw, tx, p, tiles, s);
    case 32: return launch<32>(tw, tx, p, tiles, s);
    case 64: return launch<64>(tw, tx, p, tiles, s);
    default: return -3;
  }
}

}  // namespace sm
}  // namespace mb

// Dense: C[tokens, N] (bf16 or fp32) = X[tokens, K] · W[N, K]ᵀ (+ bias).  bt ∈ {16, 32, 64}: token tile.  split_k ≥ 1; with
// split_k > 1: ws fp32 [split_k · tokens · N] and counters int [4 · ⌈N/128⌉ · ⌈tokens/bt⌉] (zero on entry, zero again on exit).
extern "C" int mb_gemm_small(const void* X, const void* W, void* C, int tokens, int N, int K, long long ldx, long long ldw, long long ldc,
                             int out_fp32, const void* bias, int bt, int split_k, float* ws, int* counters, int* error_flag,
                             cudaStream_t s) {
  using namespace mb;
  if (tokens <= 0 || N <= 0) return 0;
  if (split_k > 1 && (ws == nullptr || counters == nullptr)) return -1;
  CUtensorMap tw, tx;
  int r = make_tmap_bf16_2d(&tw, W, N, K, ldw, sm::BMW, sm::BK);
  if (r) return 1000 + r;
  r = make_tmap_bf16_2d(&tx, X, tokens, K, ldx, bt, sm::BK);
  if (r) return 2000 + r;
  sm::Params p{};
  p.tokens = tokens; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.split_k = split_k < 1 ? 1 : split_k; p.ws = ws; p.counters = counters; p.error_flag = error_flag;
  const int tiles = ((N + sm::BMW - 1) / sm::BMW) * ((tokens + bt - 1) / bt) * p.split_k;
  return sm::dispatch(bt, tw, tx, p, tiles, s);
}

// Grouped (MoE): X [rows, K] expert-sorted with segments padded to `bt` rows, tile_expert[rows / bt]; W [E·N, K]; C [rows, N] bf16.
// used_rows (optional, device): rows in use — the sort's final segment offset.
extern "C" int mb_gemm_small_grouped(const void* X, const void* W, void* C, int rows, int N, int K, int num_experts, const int* tile_expert,
                                     const int* used_rows, int bt, int* error_flag, cudaStream_t s) {
  using namespace mb;
  if (rows <= 0 || N <= 0) return 0;
  if (rows % bt || N % sm::BMW) return -1;
  CUtensorMap tw, tx;
  int r = make_tmap_bf16_2d(&tw, W, static_cast<long long>(num_experts) * N, K, K, sm::BMW, sm::BK);
  if (r) return 1000 + r;
  r = make_tmap_bf16_2d(&tx, X, rows, K, K, bt, sm::BK);
  if (r) return 2000 + r;
  sm::Params p{};
  p.tokens = rows; p.N = N; p.K = K; p.C = C; p.ldc = N; p.out_fp32 = 0;
  p.tile_expert = tile_expert; p.used_rows = used_rows; p.grouped = 1; p.split_k = 1; p.error_flag = error_flag;
  const int tiles = (N / sm::BMW) * (rows / bt);
  return sm::dispatch(bt, tw, tx, p, tiles, s);
}
