// Flash attention backward on tcgen05 tensor cores (packed variable-length, causal or full, grouped-query, head_dim 128).
//
// Two kernels, both with every contraction on `tcgen05.mma` and every accumulator in tensor memory:
//
//   dK/dV kernel   CTA = 128 keys of one (sequence, kv head).  K_j and V_j stay in shared memory; the CTA walks the query
//                  heads of the group and their 64-row query blocks (Q_i, dO_i through a 2-stage TMA ring):
//                      Sᵀ  = K_j · Q_iᵀ      dPᵀ = V_j · dO_iᵀ            (TMEM, double buffered, 64 columns each)
//                      Pᵀ  = exp2(Sᵀ·scale·log2e − lse_i·log2e)          dSᵀ = Pᵀ ∘ (dPᵀ − Δ_i) · scale
//                      dV += Pᵀ · dO_i        dK += dSᵀ · Q_i             (TMEM, 128 columns each, live for the whole CTA)
//                  The transposed products put the KEY on the TMEM lane, so a softmax thread owns one key row and writes
//                  its Pᵀ / dSᵀ row (bf16, 128-byte swizzled, K-major) straight into the A operand of the next MMA; dO_i
//                  and Q_i are read a second time from the same shared-memory tile through an MN-major descriptor.
//   dQ kernel      CTA = 128 queries of one (sequence, query head); K_j, V_j blocks of 64 keys through a 2-stage ring:
//                      S = Q_i · K_jᵀ   dP = dO_i · V_jᵀ   dS = P ∘ (dP − Δ) · scale   dQ += dS · K_j
//
// Warp roles in both: warp 0 TMA producer, warp 1 MMA issue + TMEM owner, warps 2..9 softmax / dS: thread = TMEM lane, two
// warps per lane quadrant, each taking 32 of the step's 64 columns (two warps per scheduler hide each other's TMEM-load,
// shared-memory and exp latencies; the per-query lse / Δ of step t+1 are fetched while step t is computed).
// The scores of step t+1 are issued before the gradient products of step t, so the tensor pipe has work while the
// softmax warps run.  S and dP are recomputed in both kernels (7 tile products per (i, j) pair instead of 5) — the
// price of not accumulating dQ with atomics; results are deterministic.  Every barrier wait is bounded.
#include "launch.h"
#include "ptx.cuh"

namespace mb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows, int box_cols);

namespace fab {

static constexpr int D = 128;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr uint32_t kTmemCols = 512;

struct Params {
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  __nv_bfloat16* dq;    // [T, Hq, 128]
  __nv_bfloat16* dk;    // [T, Hkv, 128]
  __nv_bfloat16* dv;
  const int* cu_seqlens;
  int Hq, Hkv, total_tokens;
  float scale;
  int causal;
  int* error_flag;
};

// write 8 bf16 (one 16-byte chunk) of a 128-byte swizzled K-major row
__device__ __forceinline__ void store_chunk(uint8_t* row_base, int row, int chunk, const float (&v)[8]) {
  uint4 w;
  w.x = pack_bf16x2(v[0], v[1]);
  w.y = pack_bf16x2(v[2], v[3]);
  w.z = pack_bf16x2(v[4], v[5]);
  w.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(row_base + ((chunk ^ (row & 7)) << 4)) = w;
}

// TMEM accumulator row (32·chunks fp32 columns) → bf16 in global memory
__device__ __forceinline__ void store_acc_cols(uint32_t taddr, __nv_bfloat16* dst, bool valid, int chunks) {
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    uint32_t o[32];
    tmem_ld_32x32(taddr + c * 32, o);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
        w.y = pack_bf16x2(__uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
        w.z = pack_bf16x2(__uint_as_float(o[i + 4]), __uint_as_float(o[i + 5]));
        w.w = pack_bf16x2(__uint_as_float(o[i + 6]), __uint_as_float(o[i + 7]));
        *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
      }
    }
  }
}
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, bool valid) { store_acc_cols(taddr, dst, valid, 4); }

// =================================================================================================================
// dK / dV
// =================================================================================================================
namespace kv {

static constexpr int BKV = 128, BQ = 64;
static constexpr int kKVBytes = BKV * D * 2;      // 32 KB: two 64-column atoms of 128 rows × 128 B
static constexpr int kKVAtom = BKV * 128;         // 16 KB
static constexpr int kQBytes = BQ * D * 2;        // 16 KB: two atoms of 64 rows × 128 B
static constexpr int kQAtom = BQ * 128;           // 8 KB
static constexpr int kPBytes = BKV * BQ * 2;      // 16 KB: one atom, 128 key rows × (64 queries = 128 B)

struct Smem {
  static constexpr int k = 0;
  static constexpr int v = k + kKVBytes;
  static constexpr int q = v + kKVBytes;            // 2 stages
  static constexpr int dout = q + 2 * kQBytes;      // 2 stages
  static constexpr int p = dout + 2 * kQBytes;      // 2 stages
  static constexpr int ds = p + 2 * kPBytes;        // 2 stages
  static constexpr int stats = ds + 2 * kPBytes;    // 2 stages × 8 warps × (32 lse + 32 delta) floats: a private copy per warp
  static constexpr int bars = stats + 2 * 8 * 64 * 4;
  static constexpr int total = bars + 256;
};

__global__ void __launch_bounds__(320, 1)
flash_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                         const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.error_flag, 0, 35);
    return;
  }
  const int b = blockIdx.z, hk = blockIdx.y;
  const int seq_start = p.cu_seqlens[b], L = p.cu_seqlens[b + 1] - seq_start;
  const int kv0 = blockIdx.x * BKV;
  if (kv0 >= L) return;
  const int G = p.Hq / p.Hkv;
  const int i_lo = p.causal ? kv0 / BQ : 0;
  const int n_i = (L + BQ - 1) / BQ - i_lo;
  const int n_it = n_i * G;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::bars);
  uint64_t* kv_full = bars;             // 1
  uint64_t* q_full = bars + 1;          // 2
  uint64_t* q_empty = bars + 3;         // 2
  uint64_t* sdp_full = bars + 5;        // 2
  uint64_t* sdp_empty = bars + 7;       // 2
  uint64_t* pds_ready = bars + 9;       // 2
  uint64_t* pds_empty = bars + 11;      // 2
  uint64_t* done = bars + 13;           // 1
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 8);
      mbar_init(&pds_ready[i], 8);
      mbar_init(&pds_empty[i], 1);
    }
    mbar_init(done, 1);
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
  const uint32_t tmem_dk = tmem + 256, tmem_dv = tmem + 384;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * kKVBytes);
      tma_load_2d(smem + Smem::k, &tm_k, kv_full, hk * D, seq_start + kv0);
      tma_load_2d(smem + Smem::k + kKVAtom, &tm_k, kv_full, hk * D + 64, seq_start + kv0);
      tma_load_2d(smem + Smem::v, &tm_v, kv_full, hk * D, seq_start + kv0);
      tma_load_2d(smem + Smem::v + kKVAtom, &tm_v, kv_full, hk * D + 64, seq_start + kv0);
      for (int it = 0; it < n_it && !*abort_flag; ++it) {
        const int st = it & 1;
        const int h = hk * G + it / n_i, row = seq_start + (i_lo + it % n_i) * BQ;
        if (!mbar_wait(&q_empty[st], ((it >> 1) & 1) ^ 1)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 31); break; }
        mbar_expect_tx(&q_full[st], 2 * kQBytes);
        uint8_t* sq = smem + Smem::q + st * kQBytes;
        uint8_t* sd = smem + Smem::dout + st * kQBytes;
        tma_load_2d(sq, &tm_q, &q_full[st], h * D, row);
        tma_load_2d(sq + kQAtom, &tm_q, &q_full[st], h * D + 64, row);
        tma_load_2d(sd, &tm_do, &q_full[st], h * D, row);
        tma_load_2d(sd + kQAtom, &tm_do, &q_full[st], h * D + 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BKV, BQ, 0, 0);    // [128 keys × 64 queries] = K-major · K-major
      constexpr uint32_t idesc_g = make_idesc_bf16(BKV, D, 0, 1);     // [128 keys × 128 d] = K-major Pᵀ/dSᵀ · MN-major dO/Q
      const uint32_t k_addr = smem_u32(smem + Smem::k), v_addr = smem_u32(smem + Smem::v);
      auto issue_sdp = [&](int it) -> bool {
        const int st = it & 1;
        if (!mbar_wait(&q_full[st], (it >> 1) & 1)) return false;
        if (!mbar_wait(&sdp_empty[st], ((it >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(smem + Smem::q + st * kQBytes);
        const uint32_t d_addr = smem_u32(smem + Smem::dout + st * kQBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_bf16(tmem + st * 128, make_smem_desc_sw128(k_addr + (ks >> 2) * kKVAtom + (ks & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(q_addr + (ks >> 2) * kQAtom + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_bf16(tmem + st * 128 + 64, make_smem_desc_sw128(v_addr + (ks >> 2) * kKVAtom + (ks & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(d_addr + (ks >> 2) * kQAtom + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
        umma_commit(&sdp_full[st]);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0);
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok && !*abort_flag; ++it) {
        if (it + 1 < n_it) ok = issue_sdp(it + 1);
        if (!ok) break;
        const int st = it & 1;
        if (!mbar_wait(&pds_ready[st], (it >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_addr = smem_u32(smem + Smem::p + st * kPBytes);
        const uint32_t s_addr = smem_u32(smem + Smem::ds + st * kPBytes);
        const uint32_t q_addr = smem_u32(smem + Smem::q + st * kQBytes);
        const uint32_t d_addr = smem_u32(smem + Smem::dout + st * kQBytes);
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)       // dV += Pᵀ[128 × 64q] · dO[64q × 128d]
          umma_bf16(tmem_dv, make_smem_desc_sw128(p_addr + ks * 32, 16, 1024),
                    make_smem_desc_sw128(d_addr + ks * (16 * 128), kQAtom, 1024), idesc_g, (it | ks) != 0);
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)       // dK += dSᵀ · Q
          umma_bf16(tmem_dk, make_smem_desc_sw128(s_addr + ks * 32, 16, 1024),
                    make_smem_desc_sw128(q_addr + ks * (16 * 128), kQAtom, 1024), idesc_g, (it | ks) != 0);
        umma_commit(&q_empty[st]);
        umma_commit(&pds_empty[st]);
      }
      if (ok) umma_commit(done);
      else { *abort_flag = 1; atomicCAS(p.error_flag, 0, 32); }
    }
  } else {
    const int q4 = warp & 3;
    const int ch = (warp - 2) >> 2;               // which 32 of the step's 64 queries this warp handles
    const int row = q4 * 32 + lane;               // key row within the block = TMEM lane
    const int kpos = kv0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    bool ok = true;
    // this lane's query of the step: lse (× log2e) and delta (× scale), fetched one step ahead
    auto fetch = [&](int it, float& l2, float& dl) {
      const int h = hk * G + it / n_i, qpos = (i_lo + it % n_i) * BQ + ch * 32 + lane;
      l2 = 0.f; dl = 0.f;
      if (it < n_it && qpos < L) {
        const long long at = static_cast<long long>(h) * p.total_tokens + seq_start + qpos;
        l2 = p.lse[at] * kLog2e;
        dl = p.delta[at] * p.scale;
      }
    };
    float nl2, ndl;
    fetch(0, nl2, ndl);
    for (int it = 0; it < n_it && !*abort_flag; ++it) {
      const int st = it & 1;
      const int qbase = (i_lo + it % n_i) * BQ + ch * 32;
      // every warp keeps its own copy of its 32 lse / delta values, so the softmax warps never meet at a CTA barrier (a
      // barrier has no time limit; the mbarrier waits below do)
      float* stats = reinterpret_cast<float*>(smem + Smem::stats) + (st * 8 + (warp - 2)) * 64;
      stats[lane] = nl2;
      stats[32 + lane] = ndl;
      __syncwarp();
      fetch(it + 1, nl2, ndl);
      if (!mbar_wait(&sdp_full[st], (it >> 1) & 1)) { ok = false; break; }
      if (!mbar_wait(&pds_empty[st], ((it >> 1) & 1) ^ 1)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (qbase + 32 > L) || (kv0 + BKV > L) || (p.causal && kv0 + BKV - 1 > qbase);
      uint8_t* prow = smem + Smem::p + st * kPBytes + (row >> 3) * 1024 + (row & 7) * 128;
      uint8_t* srow = smem + Smem::ds + st * kPBytes + (row >> 3) * 1024 + (row & 7) * 128;
      uint32_t s[32], dp[32];
      tmem_ld_32x32(tmem + lane_off + st * 128 + ch * 32, s);
      tmem_ld_32x32(tmem + lane_off + st * 128 + 64 + ch * 32, dp);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float pv[8], dsv[8];
        const float4 la = *reinterpret_cast<const float4*>(stats + g * 8), lb = *reinterpret_cast<const float4*>(stats + g * 8 + 4);
        const float4 da = *reinterpret_cast<const float4*>(stats + 32 + g * 8), db = *reinterpret_cast<const float4*>(stats + 32 + g * 8 + 4);
        const float l8[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
        const float d8[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float pe = exp2f(fmaf(__uint_as_float(s[g * 8 + i]), sl2, -l8[i]));
          if (need_mask) {
            const int qpos = qbase + g * 8 + i;
            if (qpos >= L || kpos >= L || (p.causal && kpos > qpos)) pe = 0.f;
          }
          pv[i] = pe;
          dsv[i] = pe * fmaf(__uint_as_float(dp[g * 8 + i]), p.scale, -d8[i]);
        }
        store_chunk(prow, row, ch * 4 + g, pv);
        store_chunk(srow, row, ch * 4 + g, dsv);
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sdp_empty[st]);
        mbar_arrive(&pds_ready[st]);
      }
    }
    if (ok && !*abort_flag && !mbar_wait(done, 0)) ok = false;
    if (!ok) {
      *abort_flag = 1;
      atomicCAS(p.error_flag, 0, 33);
    } else if (!*abort_flag) {
      tc_fence_after();
      const bool valid = kpos < L;
      const long long off = (static_cast<long long>(seq_start + kpos) * p.Hkv + hk) * D;
      if (ch == 0) store_acc_row(tmem_dk + lane_off, p.dk + off, valid);     // the two warps of a quadrant share the write-back
      else store_acc_row(tmem_dv + lane_off, p.dv + off, valid);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace kv

// =================================================================================================================
// dQ
// =================================================================================================================
namespace qq {

static constexpr int BQ = 128, BKV = 64;
static constexpr int kQBytes = BQ * D * 2;        // 32 KB
static constexpr int kQAtom = BQ * 128;           // 16 KB
static constexpr int kKVBytes = BKV * D * 2;      // 16 KB
static constexpr int kKVAtom = BKV * 128;         // 8 KB
static constexpr int kSBytes = BQ * BKV * 2;      // 16 KB: one atom, 128 query rows × (64 keys = 128 B)

struct Smem {
  static constexpr int q = 0;
  static constexpr int dout = q + kQBytes;
  static constexpr int k = dout + kQBytes;          // 2 stages
  static constexpr int v = k + 2 * kKVBytes;        // 2 stages
  static constexpr int ds = v + 2 * kKVBytes;       // 2 stages
  static constexpr int bars = ds + 2 * kSBytes;
  static constexpr int total = bars + 256;
};

__global__ void __launch_bounds__(320, 1)
flash_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.error_flag, 0, 45);
    return;
  }
  const int b = blockIdx.z, h = blockIdx.y;
  const int seq_start = p.cu_seqlens[b], L = p.cu_seqlens[b + 1] - seq_start;
  const int qb = gridDim.x - 1 - blockIdx.x;       // long (late) query blocks first
  const int q0 = qb * BQ;
  if (q0 >= L) return;
  const int hk = h / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(L, q0 + BQ) : L;
  const int n_blocks = (kv_end + BKV - 1) / BKV;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::bars);
  uint64_t* q_full = bars;              // 1
  uint64_t* kv_full = bars + 1;         // 2
  uint64_t* kv_empty = bars + 3;        // 2
  uint64_t* sdp_full = bars + 5;        // 2
  uint64_t* sdp_empty = bars + 7;       // 2
  uint64_t* ds_ready = bars + 9;        // 2
  uint64_t* ds_empty = bars + 11;       // 2
  uint64_t* done = bars + 13;           // 1
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 8);
      mbar_init(&ds_ready[i], 8);
      mbar_init(&ds_empty[i], 1);
    }
    mbar_init(done, 1);
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
  const uint32_t tmem_dq = tmem + 256;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, 2 * kQBytes);
      tma_load_2d(smem + Smem::q, &tm_q, q_full, h * D, seq_start + q0);
      tma_load_2d(smem + Smem::q + kQAtom, &tm_q, q_full, h * D + 64, seq_start + q0);
      tma_load_2d(smem + Smem::dout, &tm_do, q_full, h * D, seq_start + q0);
      tma_load_2d(smem + Smem::dout + kQAtom, &tm_do, q_full, h * D + 64, seq_start + q0);
      for (int j = 0; j < n_blocks && !*abort_flag; ++j) {
        const int st = j & 1, row = seq_start + j * BKV;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1)) { *abort_flag = 1; atomicCAS(p.error_flag, 0, 41); break; }
        mbar_expect_tx(&kv_full[st], 2 * kKVBytes);
        uint8_t* sk = smem + Smem::k + st * kKVBytes;
        uint8_t* sv = smem + Smem::v + st * kKVBytes;
        tma_load_2d(sk, &tm_k, &kv_full[st], hk * D, row);
        tma_load_2d(sk + kKVAtom, &tm_k, &kv_full[st], hk * D + 64, row);
        tma_load_2d(sv, &tm_v, &kv_full[st], hk * D, row);
        tma_load_2d(sv + kKVAtom, &tm_v, &kv_full[st], hk * D + 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_g = make_idesc_bf16(BQ, D, 0, 1);      // dQ[128 × 128d] = dS (K-major) · K_j (MN-major)
      const uint32_t q_addr = smem_u32(smem + Smem::q), d_addr = smem_u32(smem + Smem::dout);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&kv_full[st], (j >> 1) & 1)) return false;
        if (!mbar_wait(&sdp_empty[st], ((j >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + Smem::k + st * kKVBytes);
        const uint32_t v_addr = smem_u32(smem + Smem::v + st * kKVBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_bf16(tmem + st * 128, make_smem_desc_sw128(q_addr + (ks >> 2) * kQAtom + (ks & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(k_addr + (ks >> 2) * kKVAtom + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_bf16(tmem + st * 128 + 64, make_smem_desc_sw128(d_addr + (ks >> 2) * kQAtom + (ks & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(v_addr + (ks >> 2) * kKVAtom + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
        umma_commit(&sdp_full[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0);
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < n_blocks && ok && !*abort_flag; ++j) {
        if (j + 1 < n_blocks) ok = issue_sdp(j + 1);
        if (!ok) break;
        const int st = j & 1;
        if (!mbar_wait(&ds_ready[st], (j >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t s_addr = smem_u32(smem + Smem::ds + st * kSBytes);
        const uint32_t k_addr = smem_u32(smem + Smem::k + st * kKVBytes);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          umma_bf16(tmem_dq, make_smem_desc_sw128(s_addr + ks * 32, 16, 1024),
                    make_smem_desc_sw128(k_addr + ks * (16 * 128), kKVAtom, 1024), idesc_g, (j | ks) != 0);
        umma_commit(&kv_empty[st]);
        umma_commit(&ds_empty[st]);
      }
      if (ok) umma_commit(done);
      else { *abort_flag = 1; atomicCAS(p.error_flag, 0, 42); }
    }
  } else {
    const int q4 = warp & 3;
    const int ch = (warp - 2) >> 2;               // which 32 of the block's 64 keys this warp handles
    const int row = q4 * 32 + lane;
    const int qpos = q0 + row;
    const bool valid = qpos < L;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const long long at = static_cast<long long>(h) * p.total_tokens + seq_start + qpos;
    const float lse2 = valid ? p.lse[at] * kLog2e : 0.f;
    const float dsc = valid ? p.delta[at] * p.scale : 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && !*abort_flag; ++j) {
      const int st = j & 1, kv0 = j * BKV;
      if (!mbar_wait(&sdp_full[st], (j >> 1) & 1)) { ok = false; break; }
      if (!mbar_wait(&ds_empty[st], ((j >> 1) & 1) ^ 1)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (kv0 + BKV > L) || (q0 + BQ > L) || (p.causal && kv0 + BKV - 1 > q0);
      uint8_t* srow = smem + Smem::ds + st * kSBytes + (row >> 3) * 1024 + (row & 7) * 128;
      {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem + lane_off + st * 128 + ch * 32, s);
        tmem_ld_32x32(tmem + lane_off + st * 128 + 64 + ch * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float dsv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float pe = exp2f(fmaf(__uint_as_float(s[g * 8 + i]), sl2, -lse2));
            if (need_mask) {
              const int col = kv0 + ch * 32 + g * 8 + i;
              if (!valid || col >= L || (p.causal && col > qpos)) pe = 0.f;
            }
            dsv[i] = pe * fmaf(__uint_as_float(dp[g * 8 + i]), p.scale, -dsc);
          }
          store_chunk(srow, row, ch * 4 + g, dsv);
        }
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sdp_empty[st]);
        mbar_arrive(&ds_ready[st]);
      }
    }
    if (ok && !*abort_flag && !mbar_wait(done, 0)) ok = false;
    if (!ok) {
      *abort_flag = 1;
      atomicCAS(p.error_flag, 0, 43);
    } else if (!*abort_flag) {
      tc_fence_after();
      // the two warps of a quadrant write 64 columns each
      store_acc_cols(tmem_dq + lane_off + ch * 64, p.dq + (static_cast<long long>(seq_start + qpos) * p.Hq + h) * D + ch * 64, valid, 2);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace qq
}  // namespace fab
}  // namespace mb

using namespace mb;

// q [T, Hq, 128] (token stride q_stride elements), k / v [T, Hkv, 128] (strides k_stride / v_stride); dout, dq [T, Hq, 128]
// and dk, dv [T, Hkv, 128] contiguous; lse, delta [Hq, T] fp32 (delta = Σ_d dO·O, filled by the caller's pre-pass).
extern "C" int mb_flash_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                               void* dq, void* dk, void* dv, const int* cu_seqlens, int batch, int max_seqlen, int total_tokens,
                               long long q_stride, long long k_stride, long long v_stride, int Hq, int Hkv, float scale, int causal,
                               int* error_flag, cudaStream_t s) {
  if (batch == 0 || total_tokens == 0 || max_seqlen == 0) return 0;
  if (Hq % Hkv) return -1;
  const long long qc = static_cast<long long>(Hq) * fab::D, kc = static_cast<long long>(Hkv) * fab::D;
  CUtensorMap q64, q128, d64, d128, k64, k128, v64, v128;
  int rc = 0;
  if ((rc = make_tmap_bf16_2d(&q64, q, total_tokens, qc, q_stride, 64, 64))) return 1000 + rc;
  if ((rc = make_tmap_bf16_2d(&q128, q, total_tokens, qc, q_stride, 128, 64))) return 1000 + rc;
  if ((rc = make_tmap_bf16_2d(&d64, dout, total_tokens, qc, qc, 64, 64))) return 2000 + rc;
  if ((rc = make_tmap_bf16_2d(&d128, dout, total_tokens, qc, qc, 128, 64))) return 2000 + rc;
  if ((rc = make_tmap_bf16_2d(&k64, k, total_tokens, kc, k_stride, 64, 64))) return 3000 + rc;
  if ((rc = make_tmap_bf16_2d(&k128, k, total_tokens, kc, k_stride, 128, 64))) return 3000 + rc;
  if ((rc = make_tmap_bf16_2d(&v64, v, total_tokens, kc, v_stride, 64, 64))) return 4000 + rc;
  if ((rc = make_tmap_bf16_2d(&v128, v, total_tokens, kc, v_stride, 128, 64))) return 4000 + rc;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(fab::kv::flash_bwd_dkdv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fab::kv::Smem::total);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(fab::qq::flash_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fab::qq::Smem::total);
    if (e != cudaSuccess) return static_cast<int>(e);
    once = true;
  }
  fab::Params p{lse, delta, reinterpret_cast<__nv_bfloat16*>(dq), reinterpret_cast<__nv_bfloat16*>(dk),
                reinterpret_cast<__nv_bfloat16*>(dv), cu_seqlens, Hq, Hkv, total_tokens, scale, causal, error_flag};
  dim3 g_kv((max_seqlen + fab::kv::BKV - 1) / fab::kv::BKV, Hkv, batch);
  fab::kv::flash_bwd_dkdv_tc_kernel<<<g_kv, 320, fab::kv::Smem::total, s>>>(q64, d64, k128, v128, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 g_q((max_seqlen + fab::qq::BQ - 1) / fab::qq::BQ, Hq, batch);
  fab::qq::flash_bwd_dq_tc_kernel<<<g_q, 320, fab::qq::Smem::total, s>>>(q128, d128, k64, v64, p);
  return static_cast<int>(cudaGetLastError());
}
