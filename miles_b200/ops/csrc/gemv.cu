// Latency-optimised kernels for decode steps with at most 8 (dense: 16) tokens.
//
// With a handful of tokens every projection is a matrix-vector product: the time is the weight bytes over HBM bandwidth plus
// fixed latency, and the latency of a TMA/TMEM pipeline (barrier set-up, TMEM allocation, tile hand-offs, split-K
// reduction) is several times the streaming time.  These kernels have no prologue: every warp starts streaming weight
// rows with 16-byte read-only loads at once, eight loads in flight per lane.
//
// The arithmetic still runs on the tensor cores (`mma.sync.m16n8k16`, bf16 → fp32): 16 weight rows are the A operand, the
// ≤ 8 tokens are the B operand's 8 columns.  Because a dot product does not care about the order of its terms, a lane
// loads 8 CONSECUTIVE k of one row (one 16-byte load) and feeds register pairs to two MMAs; the activations are loaded
// with the same permutation of k, so no shuffle or shared-memory staging is needed.
//   lane = 4·g + t: A rows g and g+8, k ∈ [32c + 8t, 32c + 8t + 8); B column (token) g, same k
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

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
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

__device__ __forceinline__ float2 unpack2(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
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

// h = bf16(x + residual) for the lane's 8 k of one token; returns Σ h²
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

// NT: groups of 8 tokens (1 or 2).  One CTA = 16 output rows; its 8 warps take the 32-wide k chunks round-robin.
template <int NT, bool NORM>
__global__ void __launch_bounds__(kThreads) gemv_kernel(GemvParams p) {
  __shared__ float red[kWarps][NT][16][8];
  __shared__ float ssq[kWarps][NT][8];
  __shared__ float rstd_s[NT][8];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int ra = min(n0 + g, p.N - 1), rb = min(n0 + g + 8, p.N - 1);
  const bf16* wa_ptr = p.W + static_cast<long long>(ra) * p.K + t * 8;
  const bf16* wb_ptr = p.W + static_cast<long long>(rb) * p.K + t * 8;
  const int chunks = p.K / 32;
  float c[NT][4] = {};
  float ss[NT] = {};
  bool tok_ok[NT];
  const bf16* x_ptr[NT];
  const bf16* r_ptr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int tok = g + 8 * j;
    tok_ok[j] = tok < p.M;
    x_ptr[j] = p.x + static_cast<long long>(tok_ok[j] ? tok : 0) * p.K + t * 8;
    r_ptr[j] = (NORM && p.residual != nullptr) ? p.residual + static_cast<long long>(tok_ok[j] ? tok : 0) * p.K + t * 8 : nullptr;
  }
  // static weights do not depend on the previous kernel: their first loads are issued before the dependency wait
  constexpr int U = 8;
  if (!p.static_w) pdl_wait();
  for (int c0 = warp; c0 < chunks; c0 += kWarps * U) {
    uint4 wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ch = c0 + u * kWarps;
      if (ch < chunks) {
        wa[u] = ld_stream(wa_ptr + ch * 32);
        wb[u] = ld_stream(wb_ptr + ch * 32);
      }
    }
    if (c0 == warp && p.static_w) pdl_wait();
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ch = c0 + u * kWarps;
      if (ch < chunks) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (tok_ok[j]) {
            xv = *reinterpret_cast<const uint4*>(x_ptr[j] + ch * 32);
            if (NORM) {
              if (r_ptr[j] != nullptr) {
                const uint4 rv = *reinterpret_cast<const uint4*>(r_ptr[j] + ch * 32);
                ss[j] += add_residual(xv, rv);
                if (p.res_out != nullptr && blockIdx.x == 0)
                  *reinterpret_cast<uint4*>(p.res_out + static_cast<long long>(g + 8 * j) * p.K + ch * 32 + t * 8) = xv;
              } else {
                ss[j] += sumsq8(xv);
              }
              const uint4 nw = *reinterpret_cast<const uint4*>(p.norm_w + ch * 32 + t * 8);
              xv = scale8(xv, nw, 1.f);
            }
          }
          mma_pair(c[j], wa[u], wb[u], xv);
        }
      }
    }
  }
  if (chunks <= warp && p.static_w) pdl_wait();
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][j][g][2 * t] = c[j][0];
    red[warp][j][g][2 * t + 1] = c[j][1];
    red[warp][j][g + 8][2 * t] = c[j][2];
    red[warp][j][g + 8][2 * t + 1] = c[j][3];
    if (NORM) {
      float s = ss[j];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (t == 0) ssq[warp][j][g] = s;
    }
  }
  __syncthreads();
  if (NORM) {
    if (threadIdx.x < NT * 8) {
      const int j = threadIdx.x >> 3, tk = threadIdx.x & 7;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += ssq[w][j][tk];
      rstd_s[j][tk] = rsqrtf(s / p.K + p.eps);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < NT * 128; i += kThreads) {
    const int j = i >> 7, tk = (i >> 4) & 7, row = i & 15;
    const int tok = tk + 8 * j, n = n0 + row;
    if (tok < p.M && n < p.N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[w][j][row][tk];
      if (NORM) s *= rstd_s[j][tk];
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
      *reinterpret_cast<uint4*>(p.xn_out + static_cast<long long>(tok) * p.K + kv) = scale8(xv, nw, rstd_s[tok >> 3][tok & 7]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// MoE for ≤ 8 tokens (≤ 64 (token, choice) pairs).  No sort, gather or combine kernels: every warp holds the pair → expert
// table in two registers per lane and finds "the first pair of each distinct expert" and "the pair of (expert, token)"
// with ballots.
// ---------------------------------------------------------------------------------------------
static constexpr int kMaxPairs = 64;

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
// of the expert for all tokens and stores silu(gate) · up for the tokens routed to it.
__global__ void __launch_bounds__(kThreads) moe_gemv_up_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w13,
                                                               const int* __restrict__ topk_idx, bf16* __restrict__ act, int T, int k,
                                                               int E, int offset, int H, int F) {
  __shared__ float red[kWarps][16][8];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_pairs = T * k;
  const PairIdx pi = load_pairs(topk_idx, n_pairs, E, offset);
  // bit p of `firsts`: pair p is the first pair of its (local) expert — one bit per distinct expert of the step
  unsigned long long firsts = 0ull;
  for (int p = 0; p < n_pairs; ++p) {
    const int e = expert_of(pi, p);
    if (e >= 0 && is_first(match_mask(pi, e), p)) firsts |= 1ull << p;
  }
  const int nfb = F / 8;
  const int n_items = __popcll(firsts) * nfb;
  const bool tok_ok = g < T;
  const bf16* x_ptr = x + static_cast<long long>(tok_ok ? g : 0) * H + t * 8;
  const int chunks = H / 32;
  constexpr int U = 8;
  // work item = (distinct expert s, block of 8 features); consecutive CTAs take consecutive feature blocks of one expert
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
  const int s = item / nfb;
  unsigned long long rest = firsts;
  for (int i = 0; i < s; ++i) rest &= rest - 1ull;
  const int p = __ffsll(static_cast<long long>(rest)) - 1;
  const int e = expert_of(pi, p);
  const unsigned long long mask = match_mask(pi, e);
  const int f0 = (item % nfb) * 8;
  const bf16* base = w13 + static_cast<long long>(e) * 2 * F * H;
  const bf16* wa_ptr = base + static_cast<long long>(f0 + g) * H + t * 8;
  const bf16* wb_ptr = base + static_cast<long long>(F + f0 + g) * H + t * 8;
  float c[4] = {};
  for (int c0 = warp; c0 < chunks; c0 += kWarps * U) {
    uint4 wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ch = c0 + u * kWarps;
      if (ch < chunks) {
        wa[u] = ld_stream(wa_ptr + ch * 32);
        wb[u] = ld_stream(wb_ptr + ch * 32);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ch = c0 + u * kWarps;
      if (ch < chunks) {
        const uint4 xv = tok_ok ? *reinterpret_cast<const uint4*>(x_ptr + ch * 32) : make_uint4(0, 0, 0, 0);
        mma_pair(c, wa[u], wb[u], xv);
      }
    }
  }
  red[warp][g][2 * t] = c[0];
  red[warp][g][2 * t + 1] = c[1];
  red[warp][g + 8][2 * t] = c[2];
  red[warp][g + 8][2 * t + 1] = c[3];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int f = threadIdx.x & 7, tok = threadIdx.x >> 3;
    const int pair = tok < T ? pair_of(mask, tok, k) : -1;
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
}

// grid (H/16): CTA hb accumulates rows h0..h0+15 of the output over all experts of the step; warp w looks at pairs w, w+8, …
// and works on those that are the first pair of their expert.
// out[t, h] = Σ_experts gate_w(t, e) · (W2[e][h, :] · act[pair(t, e), :])
__global__ void __launch_bounds__(kThreads) moe_gemv_down_kernel(const bf16* __restrict__ act, const bf16* __restrict__ w2,
                                                                 const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                                 bf16* __restrict__ out, int T, int k, int E, int offset, int H, int F) {
  __shared__ float red[kWarps][16][8];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h0 = blockIdx.x * 16;
  const int chunks = F / 32;
  const int n_pairs = T * k;
  const PairIdx pi = load_pairs(topk_idx, n_pairs, E, offset);
  float c[4] = {};
  constexpr int U = 8;
  for (int p = warp; p < n_pairs; p += kWarps) {
    const int e = expert_of(pi, p);
    if (e < 0) continue;
    const unsigned long long mask = match_mask(pi, e);
    if (!is_first(mask, p)) continue;
    const int pair = g < T ? pair_of(mask, g, k) : -1;
    const float gw = pair >= 0 ? topk_w[pair] : 0.f;
    const bf16* base = w2 + static_cast<long long>(e) * H * F;
    const bf16* wa_ptr = base + static_cast<long long>(h0 + g) * F + t * 8;
    const bf16* wb_ptr = base + static_cast<long long>(h0 + g + 8) * F + t * 8;
    const bf16* a_ptr = act + static_cast<long long>(pair >= 0 ? pair : 0) * F + t * 8;
    float cs[4] = {};
    for (int c0 = 0; c0 < chunks; c0 += U) {
      uint4 wa[U], wb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (c0 + u < chunks) {
          wa[u] = ld_stream(wa_ptr + (c0 + u) * 32);
          wb[u] = ld_stream(wb_ptr + (c0 + u) * 32);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (c0 + u < chunks) {
          const uint4 xv = pair >= 0 ? *reinterpret_cast<const uint4*>(a_ptr + (c0 + u) * 32) : make_uint4(0, 0, 0, 0);
          mma_pair(cs, wa[u], wb[u], xv);
        }
      }
    }
    // accumulator columns 2t and 2t+1 are other tokens than this lane's B column: fetch their gate weights from the
    // lanes that own those tokens
    const float gw0 = __shfl_sync(0xffffffffu, gw, (2 * t) * 4);
    const float gw1 = __shfl_sync(0xffffffffu, gw, (2 * t + 1) * 4);
    c[0] += gw0 * cs[0];
    c[1] += gw1 * cs[1];
    c[2] += gw0 * cs[2];
    c[3] += gw1 * cs[3];
  }
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

}  // namespace gv
}  // namespace mb

using namespace mb;
using namespace mb::gv;

// y[M, N] = norm?(x (+ residual)) · Wᵀ (+ bias).  M ≤ 16, K a multiple of 32, 16-byte aligned rows.
// norm_w != null: RMSNorm over K with weight norm_w (after adding `residual` when given) is applied to x first; res_out / xn_out
// (optional) receive bf16(x + residual) and the normalised activations.  static_w: W is a parameter (not produced by a kernel that
// may still be running), so its loads may start before the previous kernel has finished.
extern "C" int mb_gemv(const void* x, const void* residual, const void* norm_w, float eps, const void* W, const void* bias, void* y,
                       long long ldy, int out_fp32, void* res_out, void* xn_out, int M, int N, int K, int static_w, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K % 32 || K <= 0) return -1;
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
  const dim3 grid((N + 15) / 16), block(kThreads);
  cudaError_t e;
  if (norm_w != nullptr) e = M <= 8 ? launch_pdl(gemv_kernel<1, true>, grid, block, 0, s, p) : launch_pdl(gemv_kernel<2, true>, grid, block, 0, s, p);
  else e = M <= 8 ? launch_pdl(gemv_kernel<1, false>, grid, block, 0, s, p) : launch_pdl(gemv_kernel<2, false>, grid, block, 0, s, p);
  return static_cast<int>(e);
}

// MoE FFN for T ≤ 8 tokens (T·k ≤ 64): act [T·k, F] scratch, out [T, H].  F a multiple of 32 (and of 8), H a multiple of 32.
extern "C" int mb_moe_gemv(const void* x, const void* w13, const void* w2, const int* topk_idx, const float* topk_w, void* act, void* out,
                           int T, int k, int E, int expert_offset, int H, int F, cudaStream_t s) {
  if (T <= 0) return 0;
  if (T > 8 || T * k > kMaxPairs || H % 32 || F % 32) return -1;
  const int max_items = (T * k < E ? T * k : E) * (F / 8);
  const int up_grid = max_items < 2 * 148 ? max_items : 2 * 148;
  cudaError_t e = launch_pdl(moe_gemv_up_kernel, dim3(up_grid), dim3(kThreads), 0, s, reinterpret_cast<const bf16*>(x),
                             reinterpret_cast<const bf16*>(w13), topk_idx, reinterpret_cast<bf16*>(act), T, k, E, expert_offset, H, F);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = launch_pdl(moe_gemv_down_kernel, dim3(H / 16), dim3(kThreads), 0, s, reinterpret_cast<const bf16*>(act),
                 reinterpret_cast<const bf16*>(w2), topk_idx, topk_w, reinterpret_cast<bf16*>(out), T, k, E, expert_offset, H, F);
  return static_cast<int>(e);
}
