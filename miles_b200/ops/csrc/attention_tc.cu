// Flash attention forward on tcgen05 tensor cores (packed variable-length, causal, grouped-query, head_dim 128).
//
// One CTA = 128 query rows of one (sequence, query head); two CTAs are resident per SM (256 TMEM
// columns each) so that one CTA's softmax overlaps the other's tensor-core work (≈112 KB shared memory per CTA).  Warp roles:
//   warp 0      TMA: Q tile once, then K and V tiles of 64 keys, each through its own 2-stage ring
//   warp 1      MMA issue + TMEM owner: S_j = Q·K_jᵀ into one of two S buffers, O += P_j·V_j
//   warps 2..5  softmax: thread = query row (TMEM lane).  Read S_j from TMEM, online max/sum in registers, write P_j
//               (bf16, 128-byte swizzled, K-major) to shared memory, rescale O in TMEM when the running max moved
// S_{j+1} is issued before P_j·V_j, so the tensor pipe works on the next scores while the softmax warps run.
// TMEM: S0 | S1 (64 fp32 columns each) | O (128 columns).  Shared: Q 32 KB, K 2×16 KB, V 2×16 KB, P 16 KB.
// Q, K, V are read with 2-D tensor maps over [tokens, heads·128]; rows of a tile that belong to the next sequence are
// masked as keys and never stored as queries.  All barrier waits are bounded (error flag + early exit).
#include "launch.h"
#include "ptx.cuh"

namespace mb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows, int box_cols);

namespace fa {

static constexpr int BQ = 128, BKV = 64, D = 128;
static constexpr int kQBytes = BQ * D * 2;                // 32 KB: two 64-column atoms of 128 rows × 128 B
static constexpr int kQAtom = BQ * 128;                   // 16 KB
static constexpr int kKVBytes = BKV * D * 2;              // 16 KB: two 64-column atoms of 64 rows × 128 B
static constexpr int kKVAtom = BKV * 128;                 // 8 KB
static constexpr int kPBytes = BQ * BKV * 2;              // 16 KB: one atom (64 keys = 128 B per row)
static constexpr uint32_t kTmemCols = 256;
static constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  __nv_bfloat16* o;
  float* lse;
  const int* cu_seqlens;
  const int* cu_seqlens_k;     // null: keys are the queries' own sequences.  Else sequence b has keys [cu_k[b], cu_k[b+1]) and, under
                               // the causal mask, query i sees keys ≤ i + (Lk − Lq): the queries are the LAST Lq positions of the keys
                               // (a prompt continued after a cached prefix, a later chunk of a long prompt)
  int Hq, Hkv, total_tokens;
  float scale;
  int causal;
  int* error_flag;
};

struct Smem {
  static constexpr int q = 0;
  static constexpr int k = q + kQBytes;
  static constexpr int v = k + 2 * kKVBytes;
  static constexpr int p = v + 2 * kKVBytes;
  static constexpr int bars = p + kPBytes;
  static constexpr int total = bars + 256;   // the dynamic segment is declared 1024-byte aligned; checked at run time
};

__global__ void __launch_bounds__(192, 2)
flash_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {   // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.error_flag, 25);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::bars);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2
  uint64_t* p_ready = bars + 13;      // 1
  uint64_t* pv_done = bars + 14;      // 1
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int seq_start = p.cu_seqlens[b], L = p.cu_seqlens[b + 1] - seq_start;
  const int k_start = p.cu_seqlens_k != nullptr ? p.cu_seqlens_k[b] : seq_start;
  const int Lk = p.cu_seqlens_k != nullptr ? p.cu_seqlens_k[b + 1] - k_start : L;
  const int off = Lk - L;                             // causal diagonal shift (0 when keys and queries coincide)
  const int qb = gridDim.x - 1 - blockIdx.x;          // long (late) query blocks first
  const int q0 = qb * BQ;
  if (q0 >= L) return;
  const int hk = h / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? max(0, min(Lk, q0 + BQ + off)) : Lk;
  const int n_blocks = (kv_end + BKV - 1) / BKV;
  if (n_blocks <= 0) return;                          // only with fewer keys than queries (callers keep Lk ≥ Lq): nothing to attend to

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_ptr;
  const uint32_t tmem_o = tmem + 128;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, kQBytes);
      tma_load_2d(smem + Smem::q, &tm_q, q_full, h * D, seq_start + q0);
      tma_load_2d(smem + Smem::q + kQAtom, &tm_q, q_full, h * D + 64, seq_start + q0);
      for (int j = 0; j < n_blocks && !*abort_flag; ++j) {
        const int st = j & 1;
        const int row = k_start + j * BKV;
        if (!mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 21); break; }
        mbar_expect_tx(&k_full[st], kKVBytes);
        uint8_t* sk = smem + Smem::k + st * kKVBytes;
        tma_load_2d(sk, &tm_k, &k_full[st], hk * D, row);
        tma_load_2d(sk + kKVAtom, &tm_k, &k_full[st], hk * D + 64, row);
        if (!mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1)) { *abort_flag = 1; atomicExch(p.error_flag, 24); break; }
        mbar_expect_tx(&v_full[st], kKVBytes);
        uint8_t* sv = smem + Smem::v + st * kKVBytes;
        tma_load_2d(sv, &tm_v, &v_full[st], hk * D, row);          // V: [64 keys][64 d] per atom (MN-major B operand)
        tma_load_2d(sv + kKVAtom, &tm_v, &v_full[st], hk * D + 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);   // S = Q (K-major) · K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, D, 0, 1);     // O = P (K-major) · V (MN-major, N = head dim)
      const uint32_t q_addr = smem_u32(smem + Smem::q);
      const uint32_t p_addr = smem_u32(smem + Smem::p);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
        if (!mbar_wait(&s_empty[st], ((j >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + Smem::k + st * kKVBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {   // 4 K-steps of 16 elements per 64-wide atom
          umma_bf16(tmem + st * BKV, make_smem_desc_sw128(q_addr + (ks >> 2) * kQAtom + (ks & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(k_addr + (ks >> 2) * kKVAtom + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok && !*abort_flag; ++j) {
        if (j + 1 < n_blocks) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1) || !mbar_wait(p_ready, j & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + Smem::v + st * kKVBytes);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          // P: one K-major atom (64 keys).  V: MN-major, atoms of 64 head-dim columns (LBO = one atom), 16 key rows per step
          umma_bf16(tmem_o, make_smem_desc_sw128(p_addr + ks * 32, 16, 1024),
                    make_smem_desc_sw128(v_addr + ks * (16 * 128), kKVAtom, 1024), idesc_o, (j | ks) != 0);
        }
        umma_commit(&v_empty[st]);
        umma_commit(pv_done);
      }
      if (!ok) { *abort_flag = 1; atomicExch(p.error_flag, 22); }
    }
  } else {
    const int q4 = warp & 3;                  // TMEM lane quadrant
    const int row = q4 * 32 + lane;           // query row within the tile
    const int qpos = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.f;
    uint8_t* prow = smem + Smem::p + (row >> 3) * 1024 + (row & 7) * 128;
    bool ok = true;
    for (int j = 0; j < n_blocks && !*abort_flag; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&s_full[st], (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool need_mask = (kv0 + BKV > Lk) || (p.causal && kv0 + BKV > q0 + off);
      uint32_t s[2][32];
      tmem_ld_32x32(tmem + lane_off + st * BKV, s[0]);
      tmem_ld_32x32(tmem + lane_off + st * BKV + 32, s[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);       // scores are in registers: the S buffer may be overwritten
      float mx4[4] = {m_run, -INFINITY, -INFINITY, -INFINITY};   // independent chains
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(s[c][i]);
          if (need_mask) {
            const int col = kv0 + c * 32 + i;
            if (col >= Lk || (p.causal && col > qpos + off)) v = -INFINITY;
            s[c][i] = __float_as_uint(v);
          }
          mx4[i & 3] = fmaxf(mx4[i & 3], v);
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Lazy rescaling: keep the old reference maximum while the true maximum is less than 2^8 above it (P stays ≤ 256,
      // exact in the fp32 accumulator); the final O / l and the log-sum-exp are unaffected by which reference is used.
      if (m_run != -INFINITY && (mx - m_run) * sl2 <= 8.0f) mx = m_run;
      const float msc = (mx == -INFINITY) ? 0.f : mx * sl2;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run * sl2 - msc);
      // O must be stable (previous P·V finished) before it is rescaled and before P is overwritten
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        if (!__all_sync(0xffffffffu, mx == m_run)) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      // P = exp2(s·scale·log2e − max) → bf16, written as the K-major swizzled A operand
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {          // 8 columns (16 bytes) per group
          float pv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            pv[i] = exp2f(fmaf(__uint_as_float(s[c][g * 8 + i]), sl2, -msc));
            rs4[i & 3] += pv[i];
          }
          uint4 w;
          w.x = pack_bf16x2(pv[0], pv[1]);
          w.y = pack_bf16x2(pv[2], pv[3]);
          w.z = pack_bf16x2(pv[4], pv[5]);
          w.w = pack_bf16x2(pv[6], pv[7]);
          const int chunk = c * 4 + g;          // 16-byte chunk index within the 128-byte row
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
        }
      }
      l_run = l_run * alpha + (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      m_run = mx;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && !*abort_flag) {
      if (!mbar_wait(pv_done, (n_blocks - 1) & 1)) ok = false;
    }
    if (!ok) {
      *abort_flag = 1;
      atomicExch(p.error_flag, 23);
    } else if (!*abort_flag) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool valid = qpos < L;
      __nv_bfloat16* orow = p.o + (static_cast<long long>(seq_start + qpos) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_off + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
          }
        }
      }
      if (valid && p.lse != nullptr)
        p.lse[static_cast<long long>(h) * p.total_tokens + seq_start + qpos] = (l_run > 0.f) ? m_run * p.scale + logf(l_run) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace fa
}  // namespace mb

using namespace mb;

// resident CTAs per SM of the forward kernel at its launch configuration (diagnostic; 2 is the design point)
extern "C" int mb_flash_fwd_tc_ctas_per_sm() {
  int n = 0;
  (void)cudaFuncSetAttribute(fa::flash_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::Smem::total);
  (void)cudaFuncSetAttribute(fa::flash_fwd_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fa::flash_fwd_tc_kernel, 192, fa::Smem::total) != cudaSuccess) return -1;
  return n;
}

// q [T, Hq, 128] (token stride q_stride elements), k/v [T, Hkv, 128]; o [T, Hq, 128] contiguous; lse [Hq, T].
// cu_seqlens_k / total_k_tokens: optional separate key sequences (null / 0: the queries' own), see Params.
extern "C" int mb_flash_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens, int batch,
                               int max_seqlen, int total_tokens, long long q_stride, long long k_stride, long long v_stride, int Hq,
                               int Hkv, float scale, int causal, int* error_flag, const int* cu_seqlens_k, int total_k_tokens,
                               cudaStream_t s) {
  if (batch == 0 || total_tokens == 0 || max_seqlen == 0) return 0;
  const int tk_rows = cu_seqlens_k != nullptr ? total_k_tokens : total_tokens;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_bf16_2d(&tq, q, total_tokens, static_cast<long long>(Hq) * fa::D, q_stride, fa::BQ, 64);
  if (rc) return 1000 + rc;
  rc = make_tmap_bf16_2d(&tk, k, tk_rows, static_cast<long long>(Hkv) * fa::D, k_stride, fa::BKV, 64);
  if (rc) return 2000 + rc;
  rc = make_tmap_bf16_2d(&tv, v, tk_rows, static_cast<long long>(Hkv) * fa::D, v_stride, fa::BKV, 64);
  if (rc) return 3000 + rc;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(fa::flash_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::Smem::total);
    if (e != cudaSuccess) return static_cast<int>(e);
    // two CTAs per SM need 2 × 113.25 KB: ask for the largest shared-memory carve-out
    e = cudaFuncSetAttribute(fa::flash_fwd_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    once = true;
  }
  fa::Params p{reinterpret_cast<__nv_bfloat16*>(o), lse, cu_seqlens, cu_seqlens_k, Hq, Hkv, total_tokens, scale, causal, error_flag};
  dim3 grid((max_seqlen + fa::BQ - 1) / fa::BQ, Hq, batch);
  fa::flash_fwd_tc_kernel<<<grid, 192, fa::Smem::total, s>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}
