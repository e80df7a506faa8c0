// MoE routing and token permutation around the grouped tcgen05 GEMMs.
//   router_topk   softmax over all experts + top-k (+ renormalisation); one warp per token
//   moe_align     counting sort of (token, slot) pairs by expert into 128-row-padded segments; no host sync:
//                 buffers are sized for the worst case and the tile → expert table tells the GEMM what to skip
//   moe_gather    x_perm[row] = x[token(row)]            (pad rows zero-filled)
//   moe_combine   out[t] = Σ_j w[t,j] · y_perm[row(t,j)]   (gather form: deterministic, no atomics)
//   moe_combine_bwd  dy_perm[row] = w · dout[token(row)],  dw[t,j] = ⟨dout[t], y_perm[row(t,j)]⟩
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"
#include "debug.cuh"
#include "pdl.cuh"

namespace mb {

typedef __nv_bfloat16 bf16;
static constexpr int kPad = 128;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
template <int EPL>  // experts per lane = E / 32
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, float* __restrict__ probs,
                                                          float* __restrict__ topk_w, int* __restrict__ topk_idx, long long T, int E,
                                                          int K, int normalize) {
  pdl_trigger();
  pdl_wait();
  const long long t = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = i * 32 + lane;
    v[i] = (e < E) ? logits[t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = wmax(mx);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
    s += v[i];
  }
  s = wsum(s);
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    v[i] *= inv;
    if (probs != nullptr && i * 32 + lane < E) probs[t * E + i * 32 + lane] = v[i];
  }
  float wsel = 0.f, mine_w = 0.f;
  int mine_i = 0;
  for (int j = 0; j < K; ++j) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = i * 32 + lane;
      if (e < E && (v[i] > bv)) { bv = v[i]; bi = e; }   // ascending e → ties keep the lower id
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    // remove the winner (unrolled compare keeps v[] in registers)
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (i * 32 + lane == bi) v[i] = -2.f;
    if (bi == 0x7fffffff) { bv = 0.f; bi = -1; }   // a row of NaNs has no winner: slot left empty (−1), never an id out of range
    wsel += bv;
    if (lane == j) { mine_w = bv; mine_i = bi; }
  }
  if (lane < K) {
    topk_idx[t * K + lane] = mine_i;
    topk_w[t * K + lane] = normalize ? mine_w / fmaxf(wsel, 1e-20f) : mine_w;
  }
}

// ---------------------------------------------------------------------------------------------
// Single-CTA counting sort.  idx[n] holds global expert ids; local expert = id − expert_offset, others skipped.
// Outputs: seg_offsets[E+1] (segments padded to `pad` rows), tile_expert[max_rows / pad], row_src[max_rows], dst_row[n].
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ idx, int n, const int* __restrict__ n_ptr, int E,
                                                         int expert_offset, int* __restrict__ seg_offsets, int* __restrict__ tile_expert,
                                                         int* __restrict__ row_src, int* __restrict__ dst_row, int max_rows, int pad) {
  extern __shared__ int sh[];  // counts[E], cursor[E], seg[E+1]
  pdl_trigger();
  pdl_wait();
  if (n_ptr != nullptr) n = min(n, *n_ptr);   // device-side entry count (expert-parallel receive buffers)
  int* counts = sh;
  int* cursor = sh + E;
  int* seg = sh + 2 * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = idx[i] - expert_offset;
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      seg[e] = off;
      off += (counts[e] + pad - 1) / pad * pad;
    }
    seg[E] = off;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) seg_offsets[e] = seg[e];
  const int max_tiles = max_rows / pad;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * pad;
    int ex = -1;
    if (row < seg[E]) {
      int lo = 0, hi = E;   // last e with seg[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
    }
    tile_expert[t] = ex;
  }
  // rows at or beyond seg[E] are never read (every consumer stops at seg[E]), so only the used prefix is cleared
  for (int r = threadIdx.x; r < seg[E] && r < max_rows; r += blockDim.x) row_src[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = idx[i] - expert_offset;
    int row = -1;
    if (e >= 0 && e < E) {
      row = seg[e] + atomicAdd(&cursor[e], 1);
      row_src[row] = i;
    }
    dst_row[i] = row;
  }
}

// x_perm[row, :] = x[row_src[row] / k, :]  (zero for pad rows inside used segments; rows ≥ total untouched)
__global__ void __launch_bounds__(256) moe_gather_kernel(const bf16* __restrict__ x, bf16* __restrict__ x_perm,
                                                         const int* __restrict__ row_src, const int* __restrict__ seg_offsets, int E,
                                                         int k, int H, int max_rows) {
  pdl_trigger();
  pdl_wait();
  const int total = seg_offsets[E];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < total && row < max_rows; row += gridDim.x) {
    const int src = row_src[row];
    uint4* dst = reinterpret_cast<uint4*>(x_perm + static_cast<long long>(row) * H);
    if (src >= 0 && dbg::in_bounds(dbg::kMoePairs, src, 201)) {
      const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<long long>(src / k) * H);
      for (int v = threadIdx.x; v < nvec; v += 256) dst[v] = s[v];
    } else {
      for (int v = threadIdx.x; v < nvec; v += 256) dst[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// out[t, :] = Σ_j w[t,j] · y_perm[dst_row[t·k+j], :]   (w == nullptr → weights 1)
// identity_rows: dst_row only says whether pair p took part (≥ 0); its row is p itself (per-pair return buffers).
__global__ void __launch_bounds__(256) moe_combine_kernel(const bf16* __restrict__ y_perm, const float* __restrict__ w,
                                                          const int* __restrict__ dst_row, bf16* __restrict__ out, long long T, int k,
                                                          int H, int identity_rows) {
  pdl_trigger();
  pdl_wait();
  const int nvec = H / 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    for (int v = threadIdx.x; v < nvec; v += 256) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; ++j) {
        int row = dst_row[t * k + j];
        if (row < 0) continue;
        if (identity_rows) row = static_cast<int>(t * k + j);
        const float wj = w ? w[t * k + j] : 1.f;
        const uint4 raw = *reinterpret_cast<const uint4*>(y_perm + static_cast<long long>(row) * H + v * 8);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(p[i]);
          acc[2 * i] += wj * f.x;
          acc[2 * i + 1] += wj * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + t * H + v * 8) = o;
    }
  }
}

// dy_perm[row] = w[flat]·dout[token];  dw[flat] = ⟨dout[token], y_perm[row]⟩   (one CTA per permuted row)
__global__ void __launch_bounds__(256) moe_combine_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ y_perm,
                                                              const float* __restrict__ w, const int* __restrict__ row_src,
                                                              const int* __restrict__ seg_offsets, int E, bf16* __restrict__ dy_perm,
                                                              float* __restrict__ dw, int k, int H, int max_rows) {
  __shared__ float red[8];
  const int total = seg_offsets[E];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < total && row < max_rows; row += gridDim.x) {
    const int flat = row_src[row];
    uint4* dst = reinterpret_cast<uint4*>(dy_perm + static_cast<long long>(row) * H);
    if (flat < 0) {
      for (int v = threadIdx.x; v < nvec; v += 256) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float wj = w[flat];
    const bf16* g = dout + static_cast<long long>(flat / k) * H;
    const bf16* y = y_perm + static_cast<long long>(row) * H;
    float dot = 0.f;
    for (int v = threadIdx.x; v < nvec; v += 256) {
      const uint4 graw = *reinterpret_cast<const uint4*>(g + v * 8);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
      uint4 yraw = make_uint4(0, 0, 0, 0);
      if (dw != nullptr) yraw = *reinterpret_cast<const uint4*>(y + v * 8);
      const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yraw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 gf = __bfloat1622float2(gp[i]);
        const float2 yf = __bfloat1622float2(yp[i]);
        dot += gf.x * yf.x + gf.y * yf.y;
        op[i] = __floats2bfloat162_rn(gf.x * wj, gf.y * wj);
      }
      dst[v] = o;
    }
    if (dw != nullptr) {
      dot = wsum(dot);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += red[i];
        dw[flat] = s;
      }
    }
  }
}

}  // namespace mb

using namespace mb;

MB_DEFINE_BOUNDS_API(mb_moe_bounds)

extern "C" int mb_router_topk(const float* logits, float* probs, float* topk_w, int* topk_idx, long long T, int E, int K,
                              int normalize, cudaStream_t s) {
  if (T == 0) return 0;
  if (E > 256 || K > 32) return -1;
  const unsigned blocks = static_cast<unsigned>((T + 7) / 8);
  const int epl = (E + 31) / 32;
  cudaError_t e;
  if (epl <= 1) e = launch_pdl(router_topk_kernel<1>, dim3(blocks), dim3(256), 0, s, logits, probs, topk_w, topk_idx, T, E, K, normalize);
  else if (epl <= 2) e = launch_pdl(router_topk_kernel<2>, dim3(blocks), dim3(256), 0, s, logits, probs, topk_w, topk_idx, T, E, K, normalize);
  else if (epl <= 4) e = launch_pdl(router_topk_kernel<4>, dim3(blocks), dim3(256), 0, s, logits, probs, topk_w, topk_idx, T, E, K, normalize);
  else e = launch_pdl(router_topk_kernel<8>, dim3(blocks), dim3(256), 0, s, logits, probs, topk_w, topk_idx, T, E, K, normalize);
  return static_cast<int>(e);
}

// pad: rows every expert segment is rounded up to (128 for the training GEMMs, 16/32/64 for the decode-sized grouped GEMM)
extern "C" int mb_moe_align_pad(const int* idx, int n, const int* n_ptr, int E, int expert_offset, int* seg_offsets, int* tile_expert,
                                int* row_src, int* dst_row, int max_rows, int pad, cudaStream_t s) {
  if (E > 2048 || pad <= 0) return -1;
  return static_cast<int>(launch_pdl(moe_align_kernel, dim3(1), dim3(1024), (3 * E + 1) * sizeof(int), s, idx, n, n_ptr, E, expert_offset,
                                     seg_offsets, tile_expert, row_src, dst_row, max_rows, pad));
}

extern "C" int mb_moe_align(const int* idx, int n, const int* n_ptr, int E, int expert_offset, int* seg_offsets, int* tile_expert,
                            int* row_src, int* dst_row, int max_rows, cudaStream_t s) {
  return mb_moe_align_pad(idx, n, n_ptr, E, expert_offset, seg_offsets, tile_expert, row_src, dst_row, max_rows, kPad, s);
}

extern "C" int mb_moe_gather(const void* x, void* x_perm, const int* row_src, const int* seg_offsets, int E, int k, int H,
                             int max_rows, cudaStream_t s) {
  if (max_rows == 0) return 0;
  if (H % 8) return -1;
  const int blocks = max_rows < 148 * 16 ? max_rows : 148 * 16;
  return static_cast<int>(launch_pdl(moe_gather_kernel, dim3(blocks), dim3(256), 0, s, reinterpret_cast<const bf16*>(x),
                                     reinterpret_cast<bf16*>(x_perm), row_src, seg_offsets, E, k, H, max_rows));
}

extern "C" int mb_moe_combine(const void* y_perm, const float* w, const int* dst_row, void* out, long long T, int k, int H,
                              int identity_rows, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  const int blocks = T < 148 * 16 ? static_cast<int>(T) : 148 * 16;
  return static_cast<int>(launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, s, reinterpret_cast<const bf16*>(y_perm), w, dst_row,
                                     reinterpret_cast<bf16*>(out), T, k, H, identity_rows));
}

extern "C" int mb_moe_combine_bwd(const void* dout, const void* y_perm, const float* w, const int* row_src, const int* seg_offsets,
                                  int E, void* dy_perm, float* dw, int k, int H, int max_rows, cudaStream_t s) {
  if (max_rows == 0) return 0;
  if (H % 8) return -1;
  const int blocks = max_rows < 148 * 16 ? max_rows : 148 * 16;
  moe_combine_bwd_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const bf16*>(dout), reinterpret_cast<const bf16*>(y_perm), w, row_src,
                                                seg_offsets, E, reinterpret_cast<bf16*>(dy_perm), dw, k, H, max_rows);
  return static_cast<int>(cudaGetLastError());
}
