// Variable-length (packed THD) causal flash attention with grouped-query heads: forward, backward, and
// decode over a paged KV cache.  Tiles are 64 query rows × 64 keys per CTA step, 4 warps, online softmax in
// registers, K/V streamed through double-buffered shared memory with cp.async, XOR-swizzled 16-byte chunks and
// ldmatrix fragment loads feeding mma.sync.m16n8k16 (bf16 in, fp32 accumulate).
//
// Backward is split into two kernels so that no gradient needs atomics:
//   dkdv: one CTA per 64-key block and KV head; loops over the query heads of the group and over query blocks
//         at or below the diagonal; works on transposed scores Sᵀ = K·Qᵀ so P ᵀ and dSᵀ are already A-fragments.
//   dq:   one CTA per 64-query block and query head; loops over key blocks.
// Both recompute P from the saved log-sum-exp; `delta = rowsum(dO ∘ O)` comes from a small pre-pass.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t s_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s_addr(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A [rows × D] bf16 tile in shared memory, 16-byte chunks XOR-swizzled by (row & 7).
template <int D>
struct Tile {
  static constexpr int kChunks = D / 8;
  __device__ static __forceinline__ int off(int row, int chunk) { return row * D + ((chunk ^ (row & 7)) << 3); }
};

// Load `rows` rows (row r ← global row g0 + r, valid when g0 + r < g_end) of width D into a swizzled tile.
template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(bf16* smem, const bf16* gbase, long long row_stride, int g0, int g_end) {
  constexpr int kChunks = D / 8;
  for (int i = threadIdx.x; i < ROWS * kChunks; i += THREADS) {
    const int r = i / kChunks, c = i % kChunks;
    const bool ok = (g0 + r) < g_end;
    const bf16* src = gbase + static_cast<long long>(ok ? (g0 + r) : g0) * row_stride + c * 8;
    cp_async16(smem + Tile<D>::off(r, c), src, ok);
  }
}

// A-operand fragments (16 rows × 16 k) from a row-major tile: rows r0.., k chunk pair kc (k = kc*16..).
template <int D>
__device__ __forceinline__ void load_a_frag(const bf16* tile, int r0, int kstep, uint32_t (&a)[4], int lane) {
  const int row = r0 + (lane & 15);
  const int chunk = kstep * 2 + (lane >> 4);
  ldsm_x4(s_addr(tile + Tile<D>::off(row, chunk)), a[0], a[1], a[2], a[3]);
}
// B-operand fragments for two adjacent n-tiles (16 n) × 16 k where B[k][n] = tile[n][k] (tile rows are n).
template <int D>
__device__ __forceinline__ void load_b_frag_nk(const bf16* tile, int n0, int kstep, uint32_t (&b)[4], int lane) {
  const int row = n0 + (lane & 7) + ((lane >> 4) << 3);
  const int chunk = kstep * 2 + ((lane >> 3) & 1);
  ldsm_x4(s_addr(tile + Tile<D>::off(row, chunk)), b[0], b[1], b[2], b[3]);  // (n0..7,k lo) (n0..7,k hi) (n8..15,k lo) (n8..15,k hi)
}
// B-operand fragments for two adjacent n-tiles where B[k][n] = tile[k][n] (tile rows are k): transposed load.
template <int D>
__device__ __forceinline__ void load_b_frag_kn(const bf16* tile, int k0, int nchunk, uint32_t (&b)[4], int lane) {
  const int row = k0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int chunk = nchunk + (lane >> 4);
  ldsm_x4_t(s_addr(tile + Tile<D>::off(row, chunk)), b[0], b[1], b[2], b[3]);  // (k lo,n0..7) (k hi,n0..7) (k lo,n8..15) (k hi,n8..15)
}

static constexpr int BQ = 64, BKV = 64, ATT_THREADS = 128;
static constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(ATT_THREADS) flash_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                                const bf16* __restrict__ v, bf16* __restrict__ o,
                                                                float* __restrict__ lse, const int* __restrict__ cu_seqlens,
                                                                long long q_stride, long long k_stride, long long v_stride,
                                                                int Hq, int Hkv, int total_tokens, float scale, int causal) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + BQ * D;        // 2 stages
  bf16* sV = sK + 2 * BKV * D;   // 2 stages
  const int b = blockIdx.z, h = blockIdx.y;
  const int seq_start = cu_seqlens[b], seq_end = cu_seqlens[b + 1];
  const int L = seq_end - seq_start;
  // heavier (later) query blocks first for better tail behaviour
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int q0 = qb * BQ;
  if (q0 >= L) return;
  const int hk = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* qg = q + static_cast<long long>(seq_start) * q_stride + h * D;
  const bf16* kg = k + static_cast<long long>(seq_start) * k_stride + hk * D;
  const bf16* vg = v + static_cast<long long>(seq_start) * v_stride + hk * D;

  const int kv_end = causal ? min(L, q0 + BQ) : L;
  const int n_blocks = (kv_end + BKV - 1) / BKV;

  load_tile<D, BQ, ATT_THREADS>(sQ, qg, q_stride, q0, L);
  load_tile<D, BKV, ATT_THREADS>(sK, kg, k_stride, 0, L);
  load_tile<D, BKV, ATT_THREADS>(sV, vg, v_stride, 0, L);
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const float sl2 = scale * kLog2e;
  const int r_lo = q0 + warp * 16 + (lane >> 2);  // this thread's two query rows: r_lo, r_lo + 8

  for (int j = 0; j < n_blocks; ++j) {
    const int st = j & 1;
    if (j + 1 < n_blocks) {
      load_tile<D, BKV, ATT_THREADS>(sK + (st ^ 1) * BKV * D, kg, k_stride, (j + 1) * BKV, L);
      load_tile<D, BKV, ATT_THREADS>(sV + (st ^ 1) * BKV * D, vg, v_stride, (j + 1) * BKV, L);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + st * BKV * D;
    const bf16* tV = sV + st * BKV * D;
    // S = Q Kᵀ : 16 rows × 64 keys per warp
    float s[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      load_a_frag<D>(sQ, warp * 16, ks, a, lane);
#pragma unroll
      for (int nt = 0; nt < BKV / 16; ++nt) {
        uint32_t bfr[4];
        load_b_frag_nk<D>(tK, nt * 16, ks, bfr, lane);
        mma16816(s[2 * nt], a, bfr[0], bfr[1]);
        mma16816(s[2 * nt + 1], a, bfr[2], bfr[3]);
      }
    }
    // mask + online softmax
    const int kv0 = j * BKV;
    const bool need_mask = (kv0 + BKV > L) || (causal && kv0 + BKV > q0 + warp * 16);
    float mx[2] = {m_i[0], m_i[1]};
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (need_mask) {
          const int col = kv0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int row = r_lo + ((e >> 1) << 3);
          if (col >= L || (causal && col > row)) s[nt][e] = -INFINITY;
        }
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float alpha[2], msc[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      msc[r] = (mx[r] == -INFINITY) ? 0.f : mx[r] * sl2;
      alpha[r] = (m_i[r] == -INFINITY) ? 0.f : exp2f(m_i[r] * sl2 - msc[r]);
      m_i[r] = mx[r];
      l_i[r] *= alpha[r];
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nt][e] * sl2 - msc[e >> 1]);
        s[nt][e] = p;
        rs[e >> 1] += p;
      }
    }
    l_i[0] += rs[0];
    l_i[1] += rs[1];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
    }
    // O += P V
#pragma unroll
    for (int kt = 0; kt < BKV / 16; ++kt) {
      uint32_t a[4] = {pack2(s[2 * kt][0], s[2 * kt][1]), pack2(s[2 * kt][2], s[2 * kt][3]),
                       pack2(s[2 * kt + 1][0], s[2 * kt + 1][1]), pack2(s[2 * kt + 1][2], s[2 * kt + 1][3])};
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t bfr[4];
        load_b_frag_kn<D>(tV, kt * 16, nc * 2, bfr, lane);
        mma16816(o_acc[2 * nc], a, bfr[0], bfr[1]);
        mma16816(o_acc[2 * nc + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }
  // finalize
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_lo + r * 8;
    if (row < L) {
      const float inv = l_i[r] > 0.f ? 1.f / l_i[r] : 0.f;
      bf16* orow = o + (static_cast<long long>(seq_start + row) * Hq + h) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<uint32_t*>(orow + i * 8 + (lane & 3) * 2) = pack2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
      }
      if ((lane & 3) == 0 && lse != nullptr)
        lse[static_cast<long long>(h) * total_tokens + seq_start + row] = (l_i[r] > 0.f) ? m_i[r] * scale + logf(l_i[r]) : -INFINITY;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// backward pre-pass: delta[h, t] = Σ_d dO[t,h,d]·O[t,h,d]
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta, int T, int Hq) {
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * Hq) return;
  const long long t = wid / Hq;
  const int h = static_cast<int>(wid % Hq);
  const bf16* a = o + (t * Hq + h) * D;
  const bf16* g = dout + (t * Hq + h) * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// ---------------------------------------------------------------------------------------------
// backward: dK, dV.  CTA = (key block, kv head, sequence); each warp owns 16 keys.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(ATT_THREADS) flash_bwd_dkdv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                                     const bf16* __restrict__ v, const bf16* __restrict__ dout,
                                                                     const float* __restrict__ lse, const float* __restrict__ delta,
                                                                     bf16* __restrict__ dk, bf16* __restrict__ dv,
                                                                     const int* __restrict__ cu_seqlens, long long q_stride,
                                                                     long long k_stride, long long v_stride, int Hq, int Hkv,
                                                                     int total_tokens, float scale, int causal) {
  constexpr int BQB = 32;  // query rows per step (keeps accumulators + score fragments within the register file)
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);
  bf16* sV = sK + BKV * D;
  bf16* sQ = sV + BKV * D;          // 2 stages × BQB rows
  bf16* sdO = sQ + 2 * BQB * D;     // 2 stages × BQB rows
  float* sLse = reinterpret_cast<float*>(sdO + 2 * BQB * D);  // 2 × BQB
  float* sDelta = sLse + 2 * BQB;                              // 2 × BQB
  const int b = blockIdx.z, hk = blockIdx.y;
  const int seq_start = cu_seqlens[b], seq_end = cu_seqlens[b + 1];
  const int L = seq_end - seq_start;
  const int kv0 = blockIdx.x * BKV;
  if (kv0 >= L) return;
  const int group = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* kg = k + static_cast<long long>(seq_start) * k_stride + hk * D;
  const bf16* vg = v + static_cast<long long>(seq_start) * v_stride + hk * D;
  load_tile<D, BKV, ATT_THREADS>(sK, kg, k_stride, kv0, L);
  load_tile<D, BKV, ATT_THREADS>(sV, vg, v_stride, kv0, L);
  cp_async_commit();

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk_acc[i][0] = dk_acc[i][1] = dk_acc[i][2] = dk_acc[i][3] = 0.f;
    dv_acc[i][0] = dv_acc[i][1] = dv_acc[i][2] = dv_acc[i][3] = 0.f;
  }
  const float sl2 = scale * kLog2e;
  const int qb_first = causal ? (kv0 / BQB) : 0;
  const int n_qb = (L + BQB - 1) / BQB;
  const int steps_per_head = n_qb - qb_first;
  const int total_steps = steps_per_head * group;

  auto issue = [&](int step, int st) {
    const int hq = hk * group + step / steps_per_head;
    const int qb = qb_first + step % steps_per_head;
    const bf16* qg = q + static_cast<long long>(seq_start) * q_stride + hq * D;
    const bf16* dog = dout + (static_cast<long long>(seq_start) * Hq + hq) * D;
    load_tile<D, BQB, ATT_THREADS>(sQ + st * BQB * D, qg, q_stride, qb * BQB, L);
    load_tile<D, BQB, ATT_THREADS>(sdO + st * BQB * D, dog, static_cast<long long>(Hq) * D, qb * BQB, L);
    if (threadIdx.x < BQB) {
      const int r = qb * BQB + threadIdx.x;
      const long long idx = static_cast<long long>(hq) * total_tokens + seq_start + r;
      sLse[st * BQB + threadIdx.x] = (r < L) ? lse[idx] : INFINITY;   // +inf → P = 0 for padded rows
      sDelta[st * BQB + threadIdx.x] = (r < L) ? delta[idx] : 0.f;
    }
    cp_async_commit();
  };

  if (total_steps > 0) issue(0, 0);
  for (int step = 0; step < total_steps; ++step) {
    const int st = step & 1;
    if (step + 1 < total_steps) {
      issue(step + 1, st ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int qb = qb_first + step % steps_per_head;
    const bf16* tQ = sQ + st * BQB * D;
    const bf16* tdO = sdO + st * BQB * D;
    const float* tl = sLse + st * BQB;
    const float* td = sDelta + st * BQB;
    // Sᵀ = K Qᵀ : 16 keys × BQB queries per warp
    float sT[BQB / 8][4], dpT[BQB / 8][4];
#pragma unroll
    for (int i = 0; i < BQB / 8; ++i) {
      sT[i][0] = sT[i][1] = sT[i][2] = sT[i][3] = 0.f;
      dpT[i][0] = dpT[i][1] = dpT[i][2] = dpT[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t ak[4], av[4];
      load_a_frag<D>(sK, warp * 16, ks, ak, lane);
      load_a_frag<D>(sV, warp * 16, ks, av, lane);
#pragma unroll
      for (int nt = 0; nt < BQB / 16; ++nt) {
        uint32_t bq[4], bd[4];
        load_b_frag_nk<D>(tQ, nt * 16, ks, bq, lane);
        load_b_frag_nk<D>(tdO, nt * 16, ks, bd, lane);
        mma16816(sT[2 * nt], ak, bq[0], bq[1]);
        mma16816(sT[2 * nt + 1], ak, bq[2], bq[3]);
        mma16816(dpT[2 * nt], av, bd[0], bd[1]);       // dPᵀ = V dOᵀ
        mma16816(dpT[2 * nt + 1], av, bd[2], bd[3]);
      }
    }
    // Pᵀ and dSᵀ (rows = keys, cols = queries)
    const int key_lo = kv0 + warp * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < BQB / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qc = nt * 8 + (lane & 3) * 2 + (e & 1);
        const int qrow = qb * BQB + qc;
        const int key = key_lo + ((e >> 1) << 3);
        float p = exp2f(sT[nt][e] * sl2 - tl[qc] * kLog2e);
        if (key >= L || qrow >= L || (causal && key > qrow)) p = 0.f;
        sT[nt][e] = p;
        dpT[nt][e] = p * (dpT[nt][e] - td[qc]) * scale;
      }
    }
    // dV += Pᵀ dO ; dK += dSᵀ Q   (k dimension = queries)
#pragma unroll
    for (int kt = 0; kt < BQB / 16; ++kt) {
      uint32_t ap[4] = {pack2(sT[2 * kt][0], sT[2 * kt][1]), pack2(sT[2 * kt][2], sT[2 * kt][3]),
                        pack2(sT[2 * kt + 1][0], sT[2 * kt + 1][1]), pack2(sT[2 * kt + 1][2], sT[2 * kt + 1][3])};
      uint32_t ad[4] = {pack2(dpT[2 * kt][0], dpT[2 * kt][1]), pack2(dpT[2 * kt][2], dpT[2 * kt][3]),
                        pack2(dpT[2 * kt + 1][0], dpT[2 * kt + 1][1]), pack2(dpT[2 * kt + 1][2], dpT[2 * kt + 1][3])};
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t bo[4], bq[4];
        load_b_frag_kn<D>(tdO, kt * 16, nc * 2, bo, lane);
        load_b_frag_kn<D>(tQ, kt * 16, nc * 2, bq, lane);
        mma16816(dv_acc[2 * nc], ap, bo[0], bo[1]);
        mma16816(dv_acc[2 * nc + 1], ap, bo[2], bo[3]);
        mma16816(dk_acc[2 * nc], ad, bq[0], bq[1]);
        mma16816(dk_acc[2 * nc + 1], ad, bq[2], bq[3]);
      }
    }
    __syncthreads();
  }
  if (total_steps == 0) cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int key = kv0 + warp * 16 + (lane >> 2) + r * 8;
    if (key < L) {
      bf16* dkr = dk + (static_cast<long long>(seq_start + key) * Hkv + hk) * D;
      bf16* dvr = dv + (static_cast<long long>(seq_start + key) * Hkv + hk) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(dkr + c) = pack2(dk_acc[i][2 * r], dk_acc[i][2 * r + 1]);
        *reinterpret_cast<uint32_t*>(dvr + c) = pack2(dv_acc[i][2 * r], dv_acc[i][2 * r + 1]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// backward: dQ.  CTA = (query block, query head, sequence); each warp owns 16 queries.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(ATT_THREADS) flash_bwd_dq_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                                   const bf16* __restrict__ v, const bf16* __restrict__ dout,
                                                                   const float* __restrict__ lse, const float* __restrict__ delta,
                                                                   bf16* __restrict__ dq, const int* __restrict__ cu_seqlens,
                                                                   long long q_stride, long long k_stride, long long v_stride,
                                                                   int Hq, int Hkv, int total_tokens, float scale, int causal) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sdO = sQ + BQ * D;
  bf16* sK = sdO + BQ * D;       // 2 stages
  bf16* sV = sK + 2 * BKV * D;   // 2 stages
  const int b = blockIdx.z, h = blockIdx.y;
  const int seq_start = cu_seqlens[b], seq_end = cu_seqlens[b + 1];
  const int L = seq_end - seq_start;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int q0 = qb * BQ;
  if (q0 >= L) return;
  const int hk = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* qg = q + static_cast<long long>(seq_start) * q_stride + h * D;
  const bf16* dog = dout + (static_cast<long long>(seq_start) * Hq + h) * D;
  const bf16* kg = k + static_cast<long long>(seq_start) * k_stride + hk * D;
  const bf16* vg = v + static_cast<long long>(seq_start) * v_stride + hk * D;
  const int kv_end = causal ? min(L, q0 + BQ) : L;
  const int n_blocks = (kv_end + BKV - 1) / BKV;
  load_tile<D, BQ, ATT_THREADS>(sQ, qg, q_stride, q0, L);
  load_tile<D, BQ, ATT_THREADS>(sdO, dog, static_cast<long long>(Hq) * D, q0, L);
  load_tile<D, BKV, ATT_THREADS>(sK, kg, k_stride, 0, L);
  load_tile<D, BKV, ATT_THREADS>(sV, vg, v_stride, 0, L);
  cp_async_commit();
  const int r_lo = q0 + warp * 16 + (lane >> 2);
  float lse_r[2], delta_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_lo + r * 8;
    const long long idx = static_cast<long long>(h) * total_tokens + seq_start + row;
    lse_r[r] = (row < L) ? lse[idx] * kLog2e : INFINITY;
    delta_r[r] = (row < L) ? delta[idx] : 0.f;
  }
  float dq_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq_acc[i][0] = dq_acc[i][1] = dq_acc[i][2] = dq_acc[i][3] = 0.f;
  const float sl2 = scale * kLog2e;
  for (int j = 0; j < n_blocks; ++j) {
    const int st = j & 1;
    if (j + 1 < n_blocks) {
      load_tile<D, BKV, ATT_THREADS>(sK + (st ^ 1) * BKV * D, kg, k_stride, (j + 1) * BKV, L);
      load_tile<D, BKV, ATT_THREADS>(sV + (st ^ 1) * BKV * D, vg, v_stride, (j + 1) * BKV, L);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + st * BKV * D;
    const bf16* tV = sV + st * BKV * D;
    float s[BKV / 8][4], dp[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t aq[4], ao[4];
      load_a_frag<D>(sQ, warp * 16, ks, aq, lane);
      load_a_frag<D>(sdO, warp * 16, ks, ao, lane);
#pragma unroll
      for (int nt = 0; nt < BKV / 16; ++nt) {
        uint32_t bk[4], bv[4];
        load_b_frag_nk<D>(tK, nt * 16, ks, bk, lane);
        load_b_frag_nk<D>(tV, nt * 16, ks, bv, lane);
        mma16816(s[2 * nt], aq, bk[0], bk[1]);
        mma16816(s[2 * nt + 1], aq, bk[2], bk[3]);
        mma16816(dp[2 * nt], ao, bv[0], bv[1]);
        mma16816(dp[2 * nt + 1], ao, bv[2], bv[3]);
      }
    }
    const int kv0 = j * BKV;
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = kv0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const int row = r_lo + ((e >> 1) << 3);
        float p = exp2f(s[nt][e] * sl2 - lse_r[e >> 1]);
        if (col >= L || (causal && col > row)) p = 0.f;
        s[nt][e] = p * (dp[nt][e] - delta_r[e >> 1]) * scale;   // dS
      }
    }
    // dQ += dS K
#pragma unroll
    for (int kt = 0; kt < BKV / 16; ++kt) {
      uint32_t a[4] = {pack2(s[2 * kt][0], s[2 * kt][1]), pack2(s[2 * kt][2], s[2 * kt][3]),
                       pack2(s[2 * kt + 1][0], s[2 * kt + 1][1]), pack2(s[2 * kt + 1][2], s[2 * kt + 1][3])};
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t bfr[4];
        load_b_frag_kn<D>(tK, kt * 16, nc * 2, bfr, lane);
        mma16816(dq_acc[2 * nc], a, bfr[0], bfr[1]);
        mma16816(dq_acc[2 * nc + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_lo + r * 8;
    if (row < L) {
      bf16* dqr = dq + (static_cast<long long>(seq_start + row) * Hq + h) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dqr + i * 8 + (lane & 3) * 2) = pack2(dq_acc[i][2 * r], dq_acc[i][2 * r + 1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// decode over a paged KV cache: one query token per request, split over the keys (flash-decoding).
// grid = (splits, kv head, request); a warp handles all `group` query heads of its KV head for a slice of keys,
// so every K/V row is read once per KV head.  Partial (m, l, o) are merged by `paged_merge_kernel`.
// ---------------------------------------------------------------------------------------------
template <int D, int GROUP>
__global__ void __launch_bounds__(128) paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                                                           const bf16* __restrict__ vc, const int* __restrict__ block_table,
                                                           const int* __restrict__ seq_lens, float* __restrict__ part_o,
                                                           float* __restrict__ part_ml, int max_blocks, int block_size, int Hq,
                                                           int Hkv, float scale, int num_splits) {
  const int req = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
  const int L = seq_lens[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int EPL = D / 32;  // elements per lane
  // keys of this split
  const int per = (L + num_splits - 1) / num_splits;
  const int k_begin = split * per, k_end = min(L, k_begin + per);
  float qv[GROUP][EPL];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    const bf16* qr = q + (static_cast<long long>(req) * Hq + hk * GROUP + g) * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[g][e] = __bfloat162float(qr[e]) * scale * kLog2e;
  }
  float m[GROUP], l[GROUP], acc[GROUP][EPL];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }
  const int* bt = block_table + static_cast<long long>(req) * max_blocks;
  for (int key = k_begin + warp; key < k_end; key += 4) {
    const long long slot = static_cast<long long>(bt[key / block_size]) * block_size + key % block_size;
    const bf16* kr = kc + (slot * Hkv + hk) * D + lane * EPL;
    const bf16* vr = vc + (slot * Hkv + hk) * D + lane * EPL;
    float kf[EPL], vf[EPL];
    if (EPL == 4) {
      const uint2 kk = *reinterpret_cast<const uint2*>(kr);
      const uint2 vv = *reinterpret_cast<const uint2*>(vr);
      const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kk.x));
      const float2 k1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kk.y));
      const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vv.x));
      const float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vv.y));
      kf[0] = k0.x; kf[1] = k0.y; kf[2] = k1.x; kf[3] = k1.y;
      vf[0] = v0.x; vf[1] = v0.y; vf[2] = v1.x; vf[3] = v1.y;
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) { kf[e] = __bfloat162float(kr[e]); vf[e] = __bfloat162float(vr[e]); }
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) s += qv[g][e] * kf[e];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      const float mn = fmaxf(m[g], s);
      const float a = exp2f(m[g] - mn), p = exp2f(s - mn);
      l[g] = l[g] * a + p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * a + p * vf[e];
      m[g] = mn;
    }
  }
  // merge the 4 warps through shared memory
  __shared__ float sm_m[4][GROUP], sm_l[4][GROUP];
  __shared__ float sm_o[4][GROUP][D];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][g][lane * EPL + e] = acc[g][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < GROUP * D; i += 128) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (sm_m[w][g] == -INFINITY) ? 0.f : exp2f(sm_m[w][g] - mm);
      ll += sm_l[w][g] * a;
      oo += sm_o[w][g][d] * a;
    }
    const long long base = ((static_cast<long long>(req) * Hq + hk * GROUP + g) * num_splits + split);
    part_o[base * D + d] = oo;
    if (d == 0) { part_ml[base * 2] = mm; part_ml[base * 2 + 1] = ll; }
  }
}

template <int D>
__global__ void paged_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                   int num_splits) {
  const long long rh = blockIdx.x;  // request·Hq + head
  const int d = threadIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(rh * num_splits + s) * 2]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(rh * num_splits + s) * 2];
    const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += part_ml[(rh * num_splits + s) * 2 + 1] * a;
    oo += part_o[(rh * num_splits + s) * D + d] * a;
  }
  out[rh * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
}

template <int D>
static size_t fwd_smem() { return static_cast<size_t>(BQ * D + 4 * BKV * D) * 2; }
template <int D>
static size_t dq_smem() { return static_cast<size_t>(2 * BQ * D + 4 * BKV * D) * 2; }
template <int D>
static size_t dkdv_smem() { return static_cast<size_t>(2 * BKV * D + 4 * 32 * D) * 2 + 4 * 32 * sizeof(float); }

template <typename Kern>
static int set_smem(Kern kern, size_t bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
}

}  // namespace mb

using namespace mb;

extern "C" int mb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens, int batch,
                            int max_seqlen, int total_tokens, long long q_stride, long long k_stride, long long v_stride, int Hq,
                            int Hkv, int D, float scale, int causal, cudaStream_t s) {
  if (batch == 0 || total_tokens == 0 || max_seqlen == 0) return 0;
  dim3 grid((max_seqlen + BQ - 1) / BQ, Hq, batch);
  auto Q = reinterpret_cast<const bf16*>(q);
  auto K = reinterpret_cast<const bf16*>(k);
  auto V = reinterpret_cast<const bf16*>(v);
  auto O = reinterpret_cast<bf16*>(o);
  if (D == 128) {
    static bool once = false;
    if (!once) { if (int e = set_smem(flash_fwd_kernel<128>, fwd_smem<128>())) return e; once = true; }
    flash_fwd_kernel<128><<<grid, ATT_THREADS, fwd_smem<128>(), s>>>(Q, K, V, O, lse, cu_seqlens, q_stride, k_stride, v_stride, Hq, Hkv,
                                                                    total_tokens, scale, causal);
  } else if (D == 64) {
    static bool once = false;
    if (!once) { if (int e = set_smem(flash_fwd_kernel<64>, fwd_smem<64>())) return e; once = true; }
    flash_fwd_kernel<64><<<grid, ATT_THREADS, fwd_smem<64>(), s>>>(Q, K, V, O, lse, cu_seqlens, q_stride, k_stride, v_stride, Hq, Hkv,
                                                                  total_tokens, scale, causal);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// delta[h, t] = Σ_d dO[t, h, d] · O[t, h, d] (the backward's pre-pass, shared by both backward implementations)
extern "C" int mb_attn_delta(const void* o, const void* dout, float* delta, int total_tokens, int Hq, int D, cudaStream_t s) {
  if (total_tokens == 0) return 0;
  const long long warps = static_cast<long long>(total_tokens) * Hq;
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  if (D == 128) attn_delta_kernel<128><<<blocks, 256, 0, s>>>(reinterpret_cast<const bf16*>(o), reinterpret_cast<const bf16*>(dout), delta, total_tokens, Hq);
  else if (D == 64) attn_delta_kernel<64><<<blocks, 256, 0, s>>>(reinterpret_cast<const bf16*>(o), reinterpret_cast<const bf16*>(dout), delta, total_tokens, Hq);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                            float* delta, void* dq, void* dk, void* dv, const int* cu_seqlens, int batch, int max_seqlen,
                            int total_tokens, long long q_stride, long long k_stride, long long v_stride, int Hq, int Hkv, int D,
                            float scale, int causal, cudaStream_t s) {
  if (batch == 0 || total_tokens == 0 || max_seqlen == 0) return 0;
  auto Q = reinterpret_cast<const bf16*>(q);
  auto K = reinterpret_cast<const bf16*>(k);
  auto V = reinterpret_cast<const bf16*>(v);
  auto O = reinterpret_cast<const bf16*>(o);
  auto DO = reinterpret_cast<const bf16*>(dout);
  const long long warps = static_cast<long long>(total_tokens) * Hq;
  dim3 g_kv((max_seqlen + BKV - 1) / BKV, Hkv, batch), g_q((max_seqlen + BQ - 1) / BQ, Hq, batch);
  if (D == 128) {
    static bool once = false;
    if (!once) {
      if (int e = set_smem(flash_bwd_dkdv_kernel<128>, dkdv_smem<128>())) return e;
      if (int e = set_smem(flash_bwd_dq_kernel<128>, dq_smem<128>())) return e;
      once = true;
    }
    attn_delta_kernel<128><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(O, DO, delta, total_tokens, Hq);
    flash_bwd_dkdv_kernel<128><<<g_kv, ATT_THREADS, dkdv_smem<128>(), s>>>(Q, K, V, DO, lse, delta, reinterpret_cast<bf16*>(dk),
                                                                          reinterpret_cast<bf16*>(dv), cu_seqlens, q_stride, k_stride,
                                                                          v_stride, Hq, Hkv, total_tokens, scale, causal);
    flash_bwd_dq_kernel<128><<<g_q, ATT_THREADS, dq_smem<128>(), s>>>(Q, K, V, DO, lse, delta, reinterpret_cast<bf16*>(dq), cu_seqlens,
                                                                     q_stride, k_stride, v_stride, Hq, Hkv, total_tokens, scale, causal);
  } else if (D == 64) {
    static bool once = false;
    if (!once) {
      if (int e = set_smem(flash_bwd_dkdv_kernel<64>, dkdv_smem<64>())) return e;
      if (int e = set_smem(flash_bwd_dq_kernel<64>, dq_smem<64>())) return e;
      once = true;
    }
    attn_delta_kernel<64><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(O, DO, delta, total_tokens, Hq);
    flash_bwd_dkdv_kernel<64><<<g_kv, ATT_THREADS, dkdv_smem<64>(), s>>>(Q, K, V, DO, lse, delta, reinterpret_cast<bf16*>(dk),
                                                                        reinterpret_cast<bf16*>(dv), cu_seqlens, q_stride, k_stride,
                                                                        v_stride, Hq, Hkv, total_tokens, scale, causal);
    flash_bwd_dq_kernel<64><<<g_q, ATT_THREADS, dq_smem<64>(), s>>>(Q, K, V, DO, lse, delta, reinterpret_cast<bf16*>(dq), cu_seqlens,
                                                                   q_stride, k_stride, v_stride, Hq, Hkv, total_tokens, scale, causal);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// part_o: [B·Hq·splits·D] floats, part_ml: [B·Hq·splits·2] floats
// SIMT variant (one key per warp step); `mb_paged_decode` in paged_decode.cu is the tensor-core kernel used by default.
extern "C" int mb_paged_decode_simt(const void* q, const void* kc, const void* vc, const int* block_table, const int* seq_lens, void* out,
                               float* part_o, float* part_ml, int batch, int max_blocks, int block_size, int Hq, int Hkv, int D,
                               float scale, int num_splits, cudaStream_t s) {
  if (batch == 0) return 0;
  const int group = Hq / Hkv;
  dim3 grid(num_splits, Hkv, batch);
  auto Q = reinterpret_cast<const bf16*>(q);
  auto KC = reinterpret_cast<const bf16*>(kc);
  auto VC = reinterpret_cast<const bf16*>(vc);
#define LAUNCH_DEC(DD, GG)                                                                                                   \
  paged_decode_kernel<DD, GG><<<grid, 128, 0, s>>>(Q, KC, VC, block_table, seq_lens, part_o, part_ml, max_blocks, block_size, Hq, \
                                                   Hkv, scale, num_splits)
  if (D == 128) {
    switch (group) {
      case 1: LAUNCH_DEC(128, 1); break;
      case 2: LAUNCH_DEC(128, 2); break;
      case 4: LAUNCH_DEC(128, 4); break;
      case 8: LAUNCH_DEC(128, 8); break;
      default: return -2;
    }
    paged_merge_kernel<128><<<batch * Hq, 128, 0, s>>>(part_o, part_ml, reinterpret_cast<bf16*>(out), num_splits);
  } else if (D == 64) {
    switch (group) {
      case 1: LAUNCH_DEC(64, 1); break;
      case 2: LAUNCH_DEC(64, 2); break;
      case 4: LAUNCH_DEC(64, 4); break;
      case 8: LAUNCH_DEC(64, 8); break;
      default: return -2;
    }
    paged_merge_kernel<64><<<batch * Hq, 64, 0, s>>>(part_o, part_ml, reinterpret_cast<bf16*>(out), num_splits);
  } else {
    return -1;
  }
#undef LAUNCH_DEC
  return static_cast<int>(cudaGetLastError());
}
