// Latency-optimised kernels for decode steps with at most 8 (dense: 16) tokens.
//
// With a handful of tokens every projection is a matrix-vector product: the time is the weight bytes over HBM bandwidth plus
// fixed latency, and the latency of a TMA/TMEM pipeline (barrier set-up, TMEM allocation, tile hand-offs, split-K
// reduction) is several times the streaming time.  These kernels have no such prologue:
//
//   * every thread streams ITS OWN 16-byte pieces of the weight rows through a private ring in shared memory with
//     `cp.async` (S stages of two pieces in flight per thread, no registers held, no barrier: a thread only ever reads
//     back what it copied itself), so each SM keeps 64–96 KB of weight loads in flight from the first instruction on;
//   * the activations (≤ 16 rows) are staged once per CTA in shared memory while the first weight loads fly — with the
//     residual add, the RMSNorm statistics and the norm weight applied on the way when the norm is fused;
//   * the arithmetic runs on the tensor cores (`mma.sync.m16n8k16`, bf16 → fp32): 16 weight rows are the A operand, the
//     ≤ 8 tokens the B operand's 8 columns.  A dot product does not care about the order of its terms, so a lane loads 8
//     CONSECUTIVE k of a row (one 16-byte piece) and feeds register pairs to two MMAs; the activations use the same
//     permutation of k.   lane = 4·g + t: A rows g and g+8, k ∈ [32c + 8t, 32c + 8t + 8); B column (token) g, same k.
//
//   gemv            y[M, N] = norm?(x (+ residual)) · W[N, K]ᵀ (+ bias)       M ≤ 16; optional fused add + RMSNorm prologue
//   moe_gemv_up     act[pair, F] = silu(W13[e][:F] x) · (W13[e][F:] x)        per distinct expert of the step, T ≤ 8 tokens
//   moe_gemv_down   out[T, H] = Σ_experts gate_w · W2[e] · act                 accumulated over experts in registers
#include <cuda_bf16.h>

#include "launch.h"
#include "pdl.cuh"

namespace mb {
namespace gv {

using bf16 = __nv_bfloat16;
static constexpr int kWarps = 8;
static constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// the calling thread's slot of the weight ring: [stage][row g | row g+8][thread] × 16 bytes (conflict-free both ways)
__device__ __forceinline__ uint32_t ring_slot(uint32_t ring, int stage, int which) {
  return ring + (((((stage << 1) + which) * kThreads) + threadIdx.x) << 4);
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// rows wa (row g) and wb (row g+8), activations xv: two MMAs cover the lane's 8 k
__device__ __forceinline__ void mma_pair(float (&c)[4], const uint4& wa, const uint4& wb, const uint4& xv) {
  mma_bf16(c, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
  mma_bf16(c, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
}

__device__ __forceinline__ float2 unpack2(uint32_t v) { return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// h = bf16(x + residual) for 8 elements; returns Σ h²
__device__ __forceinline__ float add_residual(uint4& xv, const uint4& rv) {
  float ss = 0.f;
  uint32_t* xs = &xv.x;
  const uint32_t* rs = &rv.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = unpack2(xs[i]), b = unpack2(rs[i]);
    xs[i] = pack2(a.x + b.x, a.y + b.y);
    const float2 h = unpack2(xs[i]);
    ss += h.x * h.x + h.y * h.y;
  }
  return ss;
}
__device__ __forceinline__ float sumsq8(const uint4& xv) {
  float ss = 0.f;
  const uint32_t* xs = &xv.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 h = unpack2(xs[i]);
    ss += h.x * h.x + h.y * h.y;
  }
  return ss;
}
__device__ __forceinline__ uint4 scale8(const uint4& xv, const uint4& wv, float s) {
  uint4 o;
  const uint32_t* xs = &xv.x;
  const uint32_t* ws = &wv.x;
  uint32_t* os = &o.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = unpack2(xs[i]), w = unpack2(ws[i]);
    os[i] = pack2(a.x * s * w.x, a.y * s * w.y);
  }
  return o;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Row stride of activations staged in shared memory: ≡ 64 (mod 128) bytes, so the two token rows a quarter-warp reads
// (8 lanes × 16 bytes) fall on disjoint banks.
__host__ __device__ inline int staged_stride(int K) { return K * 2 + 64; }

// Stage rows [0, rows) of a [*, K] bf16 matrix into shared memory (rows ≥ valid are zero); warp w takes rows w, w+8, ….
// NORM: h = bf16(x + residual) (block 0 also writes it to res_out), Σh² → rstd[row], the staged value is bf16(h · norm_w).
template <bool NORM>
__device__ __forceinline__ void stage_rows(uint8_t* xs, int rows, int valid, int K, const bf16* __restrict__ x,
                                           const bf16* __restrict__ residual, const bf16* __restrict__ norm_w, float eps,
                                           bf16* res_out, float* rstd) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = K / 8, stride = staged_stride(K);
  constexpr int B = 4;
  for (int r = warp; r < rows; r += kWarps) {
    uint8_t* row = xs + r * stride;
    float ss = 0.f;
    if (r < valid) {
      const bf16* xr = x + static_cast<long long>(r) * K;
      for (int v0 = lane; v0 < nv; v0 += 32 * B) {
        uint4 xb[B], rb[B], nb[B];
#pragma unroll
        for (int u = 0; u < B; ++u) {
          const int v = v0 + 32 * u;
          if (v < nv) {
            xb[u] = *reinterpret_cast<const uint4*>(xr + v * 8);
            if (NORM) {
              if (residual != nullptr) rb[u] = *reinterpret_cast<const uint4*>(residual + static_cast<long long>(r) * K + v * 8);
              nb[u] = *reinterpret_cast<const uint4*>(norm_w + v * 8);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < B; ++u) {
          const int v = v0 + 32 * u;
          if (v < nv) {
            if (NORM) {
              if (residual != nullptr) {
                ss += add_residual(xb[u], rb[u]);
                if (res_out != nullptr && blockIdx.x == 0) *reinterpret_cast<uint4*>(res_out + static_cast<long long>(r) * K + v * 8) = xb[u];
              } else {
                ss += sumsq8(xb[u]);
              }
              xb[u] = scale8(xb[u], nb[u], 1.f);
            }
            *reinterpret_cast<uint4*>(row + v * 16) = xb[u];
          }
        }
      }
    } else {
      for (int v = lane; v < nv; v += 32) *reinterpret_cast<uint4*>(row + v * 16) = make_uint4(0, 0, 0, 0);
    }
    if (NORM) {
      ss = warp_sum(ss);
      if (lane == 0) rstd[r] = rsqrtf(ss / K + eps);
    }
  }
}

// Plain copy of rows [0, valid) of a [*, K] bf16 matrix into shared memory with cp.async (every piece in flight at once, no
// registers); rows [valid, rows) are zeroed.  The caller commits the group and waits for it before the CTA barrier.
__device__ __forceinline__ void stage_rows_async(uint8_t* xs, int rows, int valid, int K, const bf16* __restrict__ x) {
  const int nv = K / 8, stride = staged_stride(K);
  for (int i = threadIdx.x; i < valid * nv; i += kThreads) {
    const int r = i / nv, v = i - r * nv;
    cp16(smem_addr(xs + r * stride + v * 16), x + static_cast<long long>(r) * K + v * 8);
  }
  for (int i = threadIdx.x; i < (rows - valid) * nv; i += kThreads) {
    const int r = valid + i / nv, v = i % nv;
    *reinterpret_cast<uint4*>(xs + r * stride + v * 16) = make_uint4(0, 0, 0, 0);
  }
}

struct GemvParams {
  const bf16* x;          // [M, K]
  const bf16* residual;   // [M, K] or null (NORM only)
  const bf16* norm_w;     // [K] (NORM only)
  float eps;
  const bf16* W;          // [N, K]
  const bf16* bias;       // [N] or null
  void* y;                // [M, ldy] bf16 or fp32
  long long ldy;
  int out_fp32;
  bf16* res_out;          // [M, K] or null: bf16(x + residual), written by block 0
  bf16* xn_out;           // [M, K] or null: the normalised activations, written by block 0
  int M, N, K;
  int static_w;           // W is not written by a kernel that may still run: its first loads go before the dependency wait
};

// NT: groups of 8 tokens (1 or 2); S: ring stages.  One CTA = 16 output rows; its 8 warps take the 32-wide k chunks round-robin.
template <int NT, bool NORM, int S>
__global__ void __launch_bounds__(kThreads) gemv_kernel(GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[kWarps][NT][16][8];
  __shared__ float rstd_s[NT * 8];
  pdl_trigger();
  const uint32_t ring = smem_addr(smem);
  uint8_t* xs = smem + S * 2 * kThreads * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int ra = min(n0 + g, p.N - 1), rb = min(n0 + g + 8, p.N - 1);
  const bf16* wa_ptr = p.W + static_cast<long long>(ra) * p.K + t * 8;
  const bf16* wb_ptr = p.W + static_cast<long long>(rb) * p.K + t * 8;
  const int chunks = p.K / 32;
  const int n_i = chunks > warp ? (chunks - warp + kWarps - 1) / kWarps : 0;   // this warp's chunks: warp, warp + 8, …
  auto issue = [&](int i) {
    if (i < n_i) {
      const int ch = warp + i * kWarps;
      cp16(ring_slot(ring, i & (S - 1), 0), wa_ptr + ch * 32);
      cp16(ring_slot(ring, i & (S - 1), 1), wb_ptr + ch * 32);
    }
    cp_commit();
  };
  if (!p.static_w) pdl_wait();
#pragma unroll
  for (int i = 0; i < S; ++i) issue(i);
  if (p.static_w) pdl_wait();          // static weights: their first loads are already in flight
  if (NORM) {
    stage_rows<true>(xs, NT * 8, p.M, p.K, p.x, p.residual, p.norm_w, p.eps, p.res_out, rstd_s);
  } else {
    stage_rows_async(xs, NT * 8, p.M, p.K, p.x);
    cp_commit();
    cp_wait<0>();
  }
  __syncthreads();
  const int stride = staged_stride(p.K);
  float c[NT][4] = {};
  for (int i = 0; i < n_i; ++i) {
    cp_wait<S - 1>();
    const int st = i & (S - 1), ch = warp + i * kWarps;
    const uint4 wa = lds16(ring_slot(ring, st, 0)), wb = lds16(ring_slot(ring, st, 1));
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + (g + 8 * j) * stride + ch * 64 + t * 16);
      mma_pair(c[j], wa, wb, xv);
    }
    issue(i + S);
  }
  cp_wait<0>();
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][j][g][2 * t] = c[j][0];
    red[warp][j][g][2 * t + 1] = c[j][1];
    red[warp][j][g + 8][2 * t] = c[j][2];
    red[warp][j][g + 8][2 * t + 1] = c[j][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < NT * 128; i += kThreads) {
    const int j = i >> 7, tk = (i >> 4) & 7, row = i & 15;
    const int tok = tk + 8 * j, n = n0 + row;
    if (tok < p.M && n < p.N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[w][j][row][tk];
      if (NORM) s *= rstd_s[tok];
      if (p.bias != nullptr) s += __bfloat162float(p.bias[n]);
      if (p.out_fp32) reinterpret_cast<float*>(p.y)[tok * p.ldy + n] = s;
      else reinterpret_cast<bf16*>(p.y)[tok * p.ldy + n] = __float2bfloat16(s);
    }
  }
  if (NORM && p.xn_out != nullptr && blockIdx.x == 0) {
    // second pass over the (cache-resident) activations: xn = bf16(h · rstd · w)
    for (int i = threadIdx.x; i < p.M * (p.K / 8); i += kThreads) {
      const int tok = i / (p.K / 8), kv = (i % (p.K / 8)) * 8;
      uint4 xv = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(tok) * p.K + kv);
      if (p.residual != nullptr) {
        const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(tok) * p.K + kv);
        add_residual(xv, rv);
      }
      const uint4 nw = *reinterpret_cast<const uint4*>(p.norm_w + kv);
      *reinterpret_cast<uint4*>(p.xn_out + static_cast<long long>(tok) * p.K + kv) = scale8(xv, nw, rstd_s[tok]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// MoE for ≤ 8 tokens (≤ 64 (token, choice) pairs).  No sort, gather or combine kernels: every warp holds the pair → expert
// table in two registers per lane and finds "the first pair of each distinct expert" and "the pair of (expert, token)"
// with ballots.
// ---------------------------------------------------------------------------------------------
static constexpr int kMaxPairs = 64;
static constexpr int kMoeStages = 8;

struct PairIdx { int lo, hi; };   // local expert of pairs `lane` and `lane + 32`; −1: no pair, or an expert of another rank

__device__ __forceinline__ PairIdx load_pairs(const int* __restrict__ topk_idx, int n_pairs, int E, int offset) {
  const int lane = threadIdx.x & 31;
  PairIdx pi;
  pi.lo = lane < n_pairs ? topk_idx[lane] - offset : -1;
  pi.hi = lane + 32 < n_pairs ? topk_idx[lane + 32] - offset : -1;
  if (pi.lo < 0 || pi.lo >= E) pi.lo = -1;
  if (pi.hi < 0 || pi.hi >= E) pi.hi = -1;
  return pi;
}
__device__ __forceinline__ int expert_of(const PairIdx& pi, int p) {
  const int lo = __shfl_sync(0xffffffffu, pi.lo, p & 31), hi = __shfl_sync(0xffffffffu, pi.hi, p & 31);
  return p < 32 ? lo : hi;
}
__device__ __forceinline__ unsigned long long match_mask(const PairIdx& pi, int e) {
  const unsigned lo = __ballot_sync(0xffffffffu, pi.lo == e), hi = __ballot_sync(0xffffffffu, pi.hi == e);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}
__device__ __forceinline__ bool is_first(unsigned long long mask, int p) { return (mask & ((1ull << p) - 1ull)) == 0ull; }
__device__ __forceinline__ int pair_of(unsigned long long mask, int tok, int k) {
  const unsigned long long sel = k >= 64 ? ~0ull : ((1ull << k) - 1ull);
  const unsigned long long m = (mask >> (tok * k)) & sel;
  return m ? tok * k + __ffsll(static_cast<long long>(m)) - 1 : -1;
}

// Persistent grid over (distinct expert, block of 8 features): an item computes gate rows f0..f0+7 and up rows F+f0..F+f0+7
// of the expert for all tokens and stores silu(gate) · up for the tokens routed to it.  A warp's weight stream runs
// across its items without a break (the ring keeps filling while the CTA reduces and stores an item).
__global__ void __launch_bounds__(kThreads) moe_gemv_up_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w13,
                                                               const int* __restrict__ topk_idx, bf16* __restrict__ act, int T, int k,
                                                               int E, int offset, int H, int F) {
  constexpr int S = kMoeStages;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[kWarps][16][8];
  __shared__ int slot_e[kMaxPairs];
  __shared__ unsigned long long slot_mask[kMaxPairs];
  __shared__ int n_slots_s;
  pdl_trigger();
  pdl_wait();
  const uint32_t ring = smem_addr(smem);
  uint8_t* xs = smem + S * 2 * kThreads * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_pairs = T * k;
  if (warp == 0) {
    // the distinct experts of the step, in order of first appearance
    const PairIdx pi = load_pairs(topk_idx, n_pairs, E, offset);
    int cnt = 0;
    if (E <= n_pairs) {
      // few local experts: one ballot pair per expert instead of a shuffle + ballot round per pair (the other warps wait
      // for this table; slots are then in expert order, which only changes which CTA takes which item)
      for (int e = 0; e < E; ++e) {
        const unsigned long long m = match_mask(pi, e);
        if (m == 0ull) continue;
        if (lane == 0) { slot_e[cnt] = e; slot_mask[cnt] = m; }
        ++cnt;
      }
    } else {
      for (int p = 0; p < n_pairs; ++p) {
        const int e = expert_of(pi, p);
        if (e < 0) continue;
        const unsigned long long m = match_mask(pi, e);
        if (!is_first(m, p)) continue;
        if (lane == 0) { slot_e[cnt] = e; slot_mask[cnt] = m; }
        ++cnt;
      }
    }
    if (lane == 0) n_slots_s = cnt;
  }
  stage_rows_async(xs, 8, T, H, x);
  cp_commit();
  cp_wait<0>();
  __syncthreads();
  const int nfb = F / 8;
  const int n_items = n_slots_s * nfb;
  const int n_mine = n_items > static_cast<int>(blockIdx.x) ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int chunks = H / 32;
  const int cpw = chunks > warp ? (chunks - warp + kWarps - 1) / kWarps : 0;     // chunks of an item taken by this warp
  const int total = n_mine * cpw;
  const int stride = staged_stride(H);
  // the copies are issued in stream order, so the (item, chunk) cursor advances incrementally: no division per copy
  int i_u = 0, i_item = blockIdx.x;
  const long long up_off = static_cast<long long>(F) * H;
  const bf16* i_base = nullptr;
  auto set_item = [&]() {
    if (i_item < n_items)
      i_base = w13 + static_cast<long long>(slot_e[i_item / nfb]) * 2 * F * H + static_cast<long long>((i_item % nfb) * 8 + g) * H + t * 8;
  };
  set_item();
  auto issue = [&](int q) {
    if (q < total) {
      const bf16* pa = i_base + (warp + i_u * kWarps) * 32;
      cp16(ring_slot(ring, q & (S - 1), 0), pa);
      cp16(ring_slot(ring, q & (S - 1), 1), pa + up_off);
      if (++i_u == cpw) { i_u = 0; i_item += gridDim.x; set_item(); }
    }
    cp_commit();
  };
#pragma unroll
  for (int q = 0; q < S; ++q) issue(q);
  int q = 0;
  for (int j = 0; j < n_mine; ++j) {
    const int item = blockIdx.x + j * gridDim.x;
    const int s = item / nfb, f0 = (item % nfb) * 8;
    float c[4] = {};
    for (int u = 0; u < cpw; ++u, ++q) {
      cp_wait<S - 1>();
      const int st = q & (S - 1), ch = warp + u * kWarps;
      const uint4 wa = lds16(ring_slot(ring, st, 0)), wb = lds16(ring_slot(ring, st, 1));
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + g * stride + ch * 64 + t * 16);
      mma_pair(c, wa, wb, xv);
      issue(q + S);
    }
    red[warp][g][2 * t] = c[0];
    red[warp][g][2 * t + 1] = c[1];
    red[warp][g + 8][2 * t] = c[2];
    red[warp][g + 8][2 * t + 1] = c[3];
    __syncthreads();
    if (threadIdx.x < 64) {
      const int f = threadIdx.x & 7, tok = threadIdx.x >> 3;
      const int pair = tok < T ? pair_of(slot_mask[s], tok, k) : -1;
      if (pair >= 0) {
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          gate += red[w][f][tok];
          up += red[w][f + 8][tok];
        }
        // the two halves are rounded to bf16 first, like the stored pre-activation of the general path
        gate = __bfloat162float(__float2bfloat16(gate));
        up = __bfloat162float(__float2bfloat16(up));
        const float a = gate / (1.f + __expf(-gate)) * up;
        act[static_cast<long long>(pair) * F + f0 + f] = __float2bfloat16(a);
      }
    }
    __syncthreads();   // `red` is reused by the next item
  }
  cp_wait<0>();
}

// grid (H/16): CTA hb accumulates rows h0..h0+15 of the output over all distinct experts of the step; its 8 warps take
// the 32-wide k chunks of EVERY expert round-robin (equal work per warp whatever the routing), a warp's weight stream runs
// across the experts without a break.
// out[t, h] = Σ_experts gate_w(t, e) · (W2[e][h, :] · act[pair(t, e), :])
__global__ void __launch_bounds__(kThreads) moe_gemv_down_kernel(const bf16* __restrict__ act, const bf16* __restrict__ w2,
                                                                 const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                                 bf16* __restrict__ out, int T, int k, int E, int offset, int H, int F) {
  constexpr int S = kMoeStages;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[kWarps][16][8];
  __shared__ int sl_e[kMaxPairs];
  __shared__ signed char sl_pair[kMaxPairs][8];
  __shared__ float sl_gw[kMaxPairs][8];
  __shared__ int n_slots_s;
  pdl_trigger();
  pdl_wait();
  const uint32_t ring = smem_addr(smem);
  uint8_t* as = smem + S * 2 * kThreads * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h0 = blockIdx.x * 16;
  const int chunks = F / 32;
  const int n_pairs = T * k;
  // all pair rows of the activations → shared memory, in flight while warp 0 builds the expert table (rows of other
  // ranks' experts are copied too and never read)
  stage_rows_async(as, n_pairs, n_pairs, F, act);
  cp_commit();
  if (warp == 0) {
    // the distinct experts of the step with, per token, the pair routed to them and its gate weight
    const PairIdx pi = load_pairs(topk_idx, n_pairs, E, offset);
    int cnt = 0;
    auto add_slot = [&](int e, unsigned long long mask) {
      if (lane < 8) {
        const int pair = lane < T ? pair_of(mask, lane, k) : -1;
        sl_pair[cnt][lane] = static_cast<signed char>(pair);
        sl_gw[cnt][lane] = pair >= 0 ? topk_w[pair] : 0.f;
      }
      if (lane == 0) sl_e[cnt] = e;
      ++cnt;
    };
    if (E <= n_pairs) {                      // few local experts: a ballot pair per expert (see moe_gemv_up_kernel)
      for (int e = 0; e < E; ++e) {
        const unsigned long long mask = match_mask(pi, e);
        if (mask != 0ull) add_slot(e, mask);
      }
    } else {
      for (int p = 0; p < n_pairs; ++p) {
        const int e = expert_of(pi, p);
        if (e < 0) continue;
        const unsigned long long mask = match_mask(pi, e);
        if (is_first(mask, p)) add_slot(e, mask);
      }
    }
    if (lane == 0) n_slots_s = cnt;
  }
  __syncthreads();
  const int cnt = n_slots_s;
  const int cpw = chunks > warp ? (chunks - warp + kWarps - 1) / kWarps : 0;      // chunks of an expert taken by this warp
  const int total = cnt * cpw;
  int i_u = 0, i_j = 0;                                         // issue cursor: (expert slot, chunk), advanced in stream order
  const long long row_off = static_cast<long long>(h0 + g) * F + t * 8;
  const bf16* i_base = cnt > 0 ? w2 + static_cast<long long>(sl_e[0]) * H * F + row_off : nullptr;
  auto issue = [&](int q) {
    if (q < total) {
      const bf16* pa = i_base + (warp + i_u * kWarps) * 32;
      cp16(ring_slot(ring, q & (S - 1), 0), pa);
      cp16(ring_slot(ring, q & (S - 1), 1), pa + 8 * F);
      if (++i_u == cpw) {
        i_u = 0;
        if (++i_j < cnt) i_base = w2 + static_cast<long long>(sl_e[i_j]) * H * F + row_off;
      }
    }
    cp_commit();
  };
#pragma unroll
  for (int q = 0; q < S; ++q) issue(q);
  cp_wait<S>();          // the activation rows (the oldest group) have landed; the weight ring keeps filling
  __syncthreads();
  const int stride = staged_stride(F);
  float c[4] = {};
  int q = 0;
  for (int j = 0; j < cnt; ++j) {
    const int pair = sl_pair[j][g];
    const uint8_t* arow = as + (pair >= 0 ? pair : 0) * stride + t * 16;
    float cs[4] = {};
    for (int u = 0; u < cpw; ++u, ++q) {
      cp_wait<S - 1>();
      const int st = q & (S - 1);
      const uint4 wa = lds16(ring_slot(ring, st, 0)), wb = lds16(ring_slot(ring, st, 1));
      const uint4 xv = pair >= 0 ? *reinterpret_cast<const uint4*>(arow + (warp + u * kWarps) * 64) : make_uint4(0, 0, 0, 0);
      mma_pair(cs, wa, wb, xv);
      issue(q + S);
    }
    // accumulator columns 2t and 2t+1 are tokens 2t and 2t+1
    const float gw0 = sl_gw[j][2 * t], gw1 = sl_gw[j][2 * t + 1];
    c[0] += gw0 * cs[0];
    c[1] += gw1 * cs[1];
    c[2] += gw0 * cs[2];
    c[3] += gw1 * cs[3];
  }
  cp_wait<0>();
  red[warp][g][2 * t] = c[0];
  red[warp][g][2 * t + 1] = c[1];
  red[warp][g + 8][2 * t] = c[2];
  red[warp][g + 8][2 * t + 1] = c[3];
  __syncthreads();
  if (threadIdx.x < 128) {
    const int row = threadIdx.x & 15, tok = threadIdx.x >> 4;
    if (tok < T) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[w][row][tok];
      out[static_cast<long long>(tok) * H + h0 + row] = __float2bfloat16(s);
    }
  }
}

template <typename K>
static cudaError_t set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

static constexpr int kDenseStages = 4;
static constexpr int kMaxSmem = 200 * 1024;

template <int NT, bool NORM>
static cudaError_t launch_gemv(const GemvParams& p, cudaStream_t s) {
  const int bytes = kDenseStages * 2 * kThreads * 16 + NT * 8 * staged_stride(p.K);
  static int configured = 0;
  if (configured < bytes) {
    cudaError_t e = set_smem(gemv_kernel<NT, NORM, kDenseStages>, kMaxSmem);
    if (e != cudaSuccess) return e;
    configured = kMaxSmem;
  }
  return launch_pdl(gemv_kernel<NT, NORM, kDenseStages>, dim3((p.N + 15) / 16), dim3(kThreads), bytes, s, p);
}

}  // namespace gv
}  // namespace mb

using namespace mb;
using namespace mb::gv;

// y[M, N] = norm?(x (+ residual)) · Wᵀ (+ bias).  M ≤ 16, K a multiple of 32 (≤ 8192 for M ≤ 8, ≤ 4096 above), 16-byte aligned rows.
// norm_w != null: RMSNorm over K with weight norm_w (after adding `residual` when given) is applied to x first; res_out / xn_out
// (optional) receive bf16(x + residual) and the normalised activations.  static_w: W is a parameter (not produced by a kernel that
// may still be running), so its loads may start before the previous kernel has finished.
extern "C" int mb_gemv(const void* x, const void* residual, const void* norm_w, float eps, const void* W, const void* bias, void* y,
                       long long ldy, int out_fp32, void* res_out, void* xn_out, int M, int N, int K, int static_w, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K % 32 || K <= 0) return -1;
  const int nt = M <= 8 ? 1 : 2;
  if (kDenseStages * 2 * kThreads * 16 + nt * 8 * staged_stride(K) > kMaxSmem) return -2;
  GemvParams p{};
  p.x = reinterpret_cast<const bf16*>(x);
  p.residual = reinterpret_cast<const bf16*>(residual);
  p.norm_w = reinterpret_cast<const bf16*>(norm_w);
  p.eps = eps;
  p.W = reinterpret_cast<const bf16*>(W);
  p.bias = reinterpret_cast<const bf16*>(bias);
  p.y = y; p.ldy = ldy; p.out_fp32 = out_fp32;
  p.res_out = reinterpret_cast<bf16*>(res_out);
  p.xn_out = reinterpret_cast<bf16*>(xn_out);
  p.M = M; p.N = N; p.K = K; p.static_w = static_w;
  cudaError_t e;
  if (norm_w != nullptr) e = nt == 1 ? launch_gemv<1, true>(p, s) : launch_gemv<2, true>(p, s);
  else e = nt == 1 ? launch_gemv<1, false>(p, s) : launch_gemv<2, false>(p, s);
  return static_cast<int>(e);
}

// MoE FFN for T ≤ 8 tokens (T·k ≤ 64): act [T·k, F] scratch, out [T, H].  H and F multiples of 32, H a multiple of 16.
extern "C" int mb_moe_gemv(const void* x, const void* w13, const void* w2, const int* topk_idx, const float* topk_w, void* act, void* out,
                           int T, int k, int E, int expert_offset, int H, int F, cudaStream_t s) {
  if (T <= 0) return 0;
  if (T > 8 || T * k > kMaxPairs || H % 32 || F % 32) return -1;
  const int ring_bytes = kMoeStages * 2 * kThreads * 16;
  const int up_bytes = ring_bytes + 8 * staged_stride(H);
  const int down_bytes = ring_bytes + T * k * staged_stride(F);
  if (up_bytes > kMaxSmem || down_bytes > kMaxSmem) return -2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = set_smem(moe_gemv_up_kernel, kMaxSmem);
    if (e == cudaSuccess) e = set_smem(moe_gemv_down_kernel, kMaxSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int max_items = (T * k < E ? T * k : E) * (F / 8);
  const int up_grid = max_items < 2 * 148 ? max_items : 2 * 148;
  cudaError_t e = launch_pdl(moe_gemv_up_kernel, dim3(up_grid), dim3(kThreads), up_bytes, s, reinterpret_cast<const bf16*>(x),
                             reinterpret_cast<const bf16*>(w13), topk_idx, reinterpret_cast<bf16*>(act), T, k, E, expert_offset, H, F);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = launch_pdl(moe_gemv_down_kernel, dim3(H / 16), dim3(kThreads), down_bytes, s, reinterpret_cast<const bf16*>(act),
                 reinterpret_cast<const bf16*>(w2), topk_idx, topk_w, reinterpret_cast<bf16*>(out), T, k, E, expert_offset, H, F);
  return static_cast<int>(e);
}
