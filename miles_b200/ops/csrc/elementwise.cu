// Memory-bound kernels: RMSNorm (+residual) fwd/bwd, SwiGLU fwd/bwd, fused per-head RMSNorm + rotary embedding
// fwd/bwd, KV-cache scatter, AdamW on a flat shard, column-sum reduction.  All use 16-byte vector accesses and
// fp32 math; grids are sized from the row count (one CTA per row, or a persistent multiple of the SM count for
// kernels that also accumulate a per-column reduction).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"
#include "debug.cuh"
#include "pdl.cuh"

namespace mb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    r = warp_sum(r);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(t.v[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm forward (optionally fused with the residual add).  H must be a multiple of 8.
//   ADD: r_new = x + residual (rounded to bf16, written to `res_out`), y = rmsnorm(r_new)·w
// ---------------------------------------------------------------------------------------------
template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                          __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H,
                                                          float eps) {
  __shared__ float sh[32];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  constexpr int MAXI = 4;  // rows up to 256·8·4 = 8192 wide stay in registers
  float vals[MAXI][8];
  float ss = 0.f;
  const int nvec = H / 8;
#pragma unroll
  for (int it = 0; it < MAXI; ++it) {
    const int v = threadIdx.x + it * 256;
    if (v < nvec) {
      load8(xr + v * 8, vals[it]);
      if (ADD) {
        float r[8];
        load8(residual + row * H + v * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[it][i] = __bfloat162float(__float2bfloat16(vals[it][i] + r[i]));
        store8(res_out + row * H + v * 8, vals[it]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += vals[it][i] * vals[it][i];
    }
  }
  for (int v = threadIdx.x + MAXI * 256; v < nvec; v += 256) {  // very wide rows: second read comes from L2
    float t[8];
    load8(xr + v * 8, t);
    if (ADD) {
      float r[8];
      load8(residual + row * H + v * 8, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) t[i] = __bfloat162float(__float2bfloat16(t[i] + r[i]));
      store8(res_out + row * H + v * 8, t);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += t[i] * t[i];
  }
  ss = block_sum<256>(ss, sh);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int it = 0; it < MAXI; ++it) {
    const int v = threadIdx.x + it * 256;
    if (v < nvec) {
      float wv[8], o[8];
      load8(w + v * 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = vals[it][i] * rstd * wv[i];
      store8(y + row * H + v * 8, o);
    }
  }
  for (int v = threadIdx.x + MAXI * 256; v < nvec; v += 256) {
    float t[8], wv[8], o[8];
    load8((ADD ? res_out : x) + row * H + v * 8, t);
    load8(w + v * 8, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = t[i] * rstd * wv[i];
    store8(y + row * H + v * 8, o);
  }
}

// The same op with one WARP per row, for rows of 256·VPL elements (VPL 16-byte vectors per lane): every lane has all of its
// loads in flight at once (2·VPL·16 bytes), the row sum needs shuffles only — no shared memory, no CTA barrier — and the
// post-add values wait in registers as packed bf16.  Eight rows per CTA.
template <bool ADD, int VPL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                                               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                               __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out,
                                                               long long T, float eps) {
  pdl_trigger();
  pdl_wait();
  constexpr int H = VPL * 256;
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (row >= T) return;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
  bf16x8 v[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) v[i] = xr[lane + 32 * i];
  if (ADD) {
    const bf16x8* rr = reinterpret_cast<const bf16x8*>(residual + row * H);
    bf16x8 r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) r[i] = rr[lane + 32 * i];
    bf16x8* ro = reinterpret_cast<bf16x8*>(res_out + row * H);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(v[i].v[j]), b = __bfloat1622float2(r[i].v[j]);
        v[i].v[j] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
      ro[lane + 32 * i] = v[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(v[i].v[j]);
      ss += a.x * a.x + a.y * a.y;
    }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / H + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * H);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const bf16x8 wv = wr[lane + 32 * i];
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(v[i].v[j]), b = __bfloat1622float2(wv.v[j]);
      o.v[j] = __floats2bfloat162_rn(a.x * rstd * b.x, a.y * rstd * b.y);
    }
    yr[lane + 32 * i] = o;
  }
}

// RMSNorm backward.  x is the normalised input (the post-add residual stream), dy the gradient of y,
// `dres` an optional extra gradient flowing into x directly (the residual branch).
//   dx = rstd·(w·dy − x̂·mean(w·dy·x̂)) + dres ;   dw_partial[block] += dy·x̂
// Persistent grid; each CTA writes one row of fp32 partial dw sums, reduced by `colsum_kernel`.
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                          const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres,
                                                          const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                          float* __restrict__ dw_partial, int T, int H) {
  __shared__ float sh[32];
  constexpr int MAXI = 4;
  const int nvec = H / 8;
  float dwacc[MAXI][8];
#pragma unroll
  for (int it = 0; it < MAXI; ++it)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[it][i] = 0.f;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[MAXI][8], g[MAXI][8];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < MAXI; ++it) {
      const int v = threadIdx.x + it * 256;
      if (v < nvec) {
        float xv[8], dv[8], wv[8];
        load8(x + row * H + v * 8, xv);
        load8(dy + row * H + v * 8, dv);
        load8(w + v * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[it][i] = xv[i] * rstd;
          g[it][i] = dv[i] * wv[i];
          dot += g[it][i] * xh[it][i];
          dwacc[it][i] += dv[i] * xh[it][i];
        }
      }
    }
    dot = block_sum<256>(dot, sh) / H;
#pragma unroll
    for (int it = 0; it < MAXI; ++it) {
      const int v = threadIdx.x + it * 256;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[it][i] - xh[it][i] * dot);
        if (dres != nullptr) {
          float r[8];
          load8(dres + row * H + v * 8, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        store8(dx + row * H + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < MAXI; ++it) {
    const int v = threadIdx.x + it * 256;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) dw_partial[static_cast<long long>(blockIdx.x) * H + v * 8 + i] = dwacc[it][i];
    }
  }
}

// out[c] = Σ_r partial[r, c]  (fp32 in, bf16 or fp32 out)
__global__ void colsum_kernel(const float* __restrict__ partial, void* __restrict__ out, int R, int C, int out_fp32) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int r = 0; r < R; ++r) s += partial[static_cast<long long>(r) * C + c];
  if (out_fp32) reinterpret_cast<float*>(out)[c] = s;
  else reinterpret_cast<__nv_bfloat16*>(out)[c] = __float2bfloat16(s);
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: in [T, 2F] (gate | up) → out [T, F]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                         long long T, int F, const int* __restrict__ rows_ptr) {
  pdl_trigger();
  pdl_wait();
  const int nvec = F / 8;
  if (rows_ptr != nullptr) T = min(T, static_cast<long long>(*rows_ptr));  // device-side row count (MoE padded buffers)
  const long long total = T * nvec;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const long long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    float g[8], u[8], o[8];
    load8(in + t * 2 * F + v * 8, g);
    load8(in + t * 2 * F + F + v * 8, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    store8(out + t * F + v * 8, o);
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                                                         __nv_bfloat16* __restrict__ din, long long T, int F,
                                                         const int* __restrict__ rows_ptr) {
  const int nvec = F / 8;
  if (rows_ptr != nullptr) T = min(T, static_cast<long long>(*rows_ptr));
  const long long total = T * nvec;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const long long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    float g[8], u[8], d[8], dg[8], du[8];
    load8(in + t * 2 * F + v * 8, g);
    load8(in + t * 2 * F + F + v * 8, u);
    load8(dout + t * F + v * 8, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      dg[k] = d[k] * u[k] * s * (1.f + g[k] * (1.f - s));
      du[k] = d[k] * g[k] * s;
    }
    store8(din + t * 2 * F + v * 8, dg);
    store8(din + t * 2 * F + F + v * 8, du);
  }
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm (optional) + NeoX rotary embedding on q and k, in one pass.  One warp per (token, head).
// Layout [T, heads, D]; pairs are (i, i + D/2).  D ∈ {64, 128}.
// ---------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void norm_rope_row(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                              const __nv_bfloat16* __restrict__ w, float pos, float log2_theta, float eps,
                                              float* rstd_out, int lane, __nv_bfloat16* __restrict__ dst2 = nullptr) {
  constexpr int EPL = D / 64;  // elements per lane in each half
  float a[EPL], b[EPL];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    a[e] = __bfloat162float(src[lane * EPL + e]);
    b[e] = __bfloat162float(src[D / 2 + lane * EPL + e]);
    ss += a[e] * a[e] + b[e] * b[e];
  }
  float rstd = 1.f;
  if (w != nullptr) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + eps);
    if (rstd_out != nullptr && lane == 0) *rstd_out = rstd;
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int j = lane * EPL + e;
    float x1 = a[e], x2 = b[e];
    if (w != nullptr) {
      x1 = __bfloat162float(__float2bfloat16(x1 * rstd * __bfloat162float(w[j])));
      x2 = __bfloat162float(__float2bfloat16(x2 * rstd * __bfloat162float(w[D / 2 + j])));
    }
    const float inv_freq = exp2f(-log2_theta * (2.f * j) / D);
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    const __nv_bfloat16 o1 = __float2bfloat16(x1 * c - x2 * s), o2 = __float2bfloat16(x2 * c + x1 * s);
    dst[j] = o1;
    dst[D / 2 + j] = o2;
    if (dst2 != nullptr) {
      dst2[j] = o1;
      dst2[D / 2 + j] = o2;
    }
  }
}

// Engine form: the same per-head norm + rotary for q and k, with the rotated k and the raw v also written into the
// paged KV cache at each token's slot (slot < 0: token not cached).  One warp per (token, q/k/v head).
template <int D>
__global__ void __launch_bounds__(256) qk_norm_rope_cache_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                                 const __nv_bfloat16* __restrict__ v, long long q_tok_stride,
                                                                 long long k_tok_stride, long long v_tok_stride,
                                                                 const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                                                 const int* __restrict__ positions, __nv_bfloat16* __restrict__ qo,
                                                                 __nv_bfloat16* __restrict__ ko, __nv_bfloat16* __restrict__ kc,
                                                                 __nv_bfloat16* __restrict__ vc, const long long* __restrict__ slots,
                                                                 long long T, int Hq, int Hk, float log2_theta, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int heads = Hq + 2 * Hk;
  if (wid >= T * heads) return;
  const long long t = wid / heads;
  const int h = static_cast<int>(wid % heads);
  if (h < Hq) {
    norm_rope_row<D>(q + t * q_tok_stride + h * D, qo + (t * Hq + h) * D, qw, static_cast<float>(positions[t]), log2_theta, eps,
                     nullptr, lane);
    return;
  }
  long long slot = slots[t];
  if (slot >= 0 && !dbg::in_bounds(dbg::kKvSlots, slot, 101)) slot = -1;   // debug build: a slot outside the cache is recorded, not written
  if (h < Hq + Hk) {
    const int hk = h - Hq;
    norm_rope_row<D>(k + t * k_tok_stride + hk * D, ko + (t * Hk + hk) * D, kw, static_cast<float>(positions[t]), log2_theta, eps,
                     nullptr, lane, slot >= 0 ? kc + (slot * Hk + hk) * D : nullptr);
  } else if (slot >= 0) {
    const int hk = h - Hq - Hk;
    constexpr int EPL = D / 32;   // 4 (8 bytes) or 2 (4 bytes) elements per lane
    const __nv_bfloat16* src = v + t * v_tok_stride + hk * D + lane * EPL;
    __nv_bfloat16* dst = vc + (slot * Hk + hk) * D + lane * EPL;
    if (EPL == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
    else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
  }
}

template <int D>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                               long long q_tok_stride, long long k_tok_stride,
                                                               const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                                               const int* __restrict__ positions, __nv_bfloat16* __restrict__ qo,
                                                               __nv_bfloat16* __restrict__ ko, float* __restrict__ q_rstd,
                                                               float* __restrict__ k_rstd, long long T, int Hq, int Hk, float log2_theta,
                                                               float eps) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int heads = Hq + Hk;
  if (wid >= T * heads) return;
  const long long t = wid / heads;
  const int h = static_cast<int>(wid % heads);
  const float pos = static_cast<float>(positions[t]);
  if (h < Hq) {
    norm_rope_row<D>(q + t * q_tok_stride + h * D, qo + (t * Hq + h) * D, qw, pos, log2_theta, eps,
                     q_rstd ? q_rstd + t * Hq + h : nullptr, lane);
  } else {
    const int hk = h - Hq;
    norm_rope_row<D>(k + t * k_tok_stride + hk * D, ko + (t * Hk + hk) * D, kw, pos, log2_theta, eps,
                     k_rstd ? k_rstd + t * Hk + hk : nullptr, lane);
  }
}

// Backward: un-rotate the incoming gradient, then the RMSNorm backward per head.  dw partial sums per CTA.
template <int D>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long x_tok_stride,
                                                               const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                                               const __nv_bfloat16* __restrict__ dy, const int* __restrict__ positions,
                                                               __nv_bfloat16* __restrict__ dx, long long dx_tok_stride,
                                                               float* __restrict__ dw_partial, long long T, int Hn, float log2_theta) {
  constexpr int EPL = D / 64;
  __shared__ float sh_dw[8][D];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  float dwa[EPL], dwb[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) dwa[e] = dwb[e] = 0.f;
  const long long nrows = T * Hn;
  for (long long r = (blockIdx.x * 256ll + threadIdx.x) >> 5; r < nrows; r += (static_cast<long long>(gridDim.x) * 256) >> 5) {
    const long long t = r / Hn;
    const int h = static_cast<int>(r % Hn);
    const float pos = static_cast<float>(positions[t]);
    const __nv_bfloat16* xr = x + t * x_tok_stride + h * D;
    const __nv_bfloat16* gr = dy + (t * Hn + h) * D;
    __nv_bfloat16* dr = dx + t * dx_tok_stride + h * D;
    float g1[EPL], g2[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int j = lane * EPL + e;
      const float inv_freq = exp2f(-log2_theta * (2.f * j) / D);
      float s, c;
      sincosf(pos * inv_freq, &s, &c);
      const float d1 = __bfloat162float(gr[j]), d2 = __bfloat162float(gr[D / 2 + j]);
      g1[e] = d1 * c + d2 * s;   // transpose of the rotation
      g2[e] = d2 * c - d1 * s;
    }
    if (w == nullptr) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        dr[lane * EPL + e] = __float2bfloat16(g1[e]);
        dr[D / 2 + lane * EPL + e] = __float2bfloat16(g2[e]);
      }
      continue;
    }
    const float rstd = rstd_in[r];
    float xa[EPL], xb[EPL], ga[EPL], gb[EPL];
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int j = lane * EPL + e;
      xa[e] = __bfloat162float(xr[j]) * rstd;
      xb[e] = __bfloat162float(xr[D / 2 + j]) * rstd;
      ga[e] = g1[e] * __bfloat162float(w[j]);
      gb[e] = g2[e] * __bfloat162float(w[D / 2 + j]);
      dot += ga[e] * xa[e] + gb[e] * xb[e];
      dwa[e] += g1[e] * xa[e];
      dwb[e] += g2[e] * xb[e];
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      dr[lane * EPL + e] = __float2bfloat16(rstd * (ga[e] - xa[e] * dot));
      dr[D / 2 + lane * EPL + e] = __float2bfloat16(rstd * (gb[e] - xb[e] * dot));
    }
  }
  if (w != nullptr && dw_partial != nullptr) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      sh_dw[wib][lane * EPL + e] = dwa[e];
      sh_dw[wib][D / 2 + lane * EPL + e] = dwb[e];
    }
    __syncthreads();
    if (threadIdx.x < D) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += sh_dw[i][threadIdx.x];
      dw_partial[static_cast<long long>(blockIdx.x) * D + threadIdx.x] = s;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding alone (NeoX pairing: element i rotates with element i + D/2), forward or inverse (= its own backward).
// One warp per (token, head); x [T, H, D] with token stride `tok_stride`, y contiguous.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                   const int* __restrict__ positions, long long T, int H, long long tok_stride,
                                                   float log2_theta, int inverse) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  if (wid >= T * H) return;
  const long long t = wid / H;
  const int h = static_cast<int>(wid % H);
  const __nv_bfloat16* src = x + t * tok_stride + static_cast<long long>(h) * D;
  __nv_bfloat16* dst = y + (t * H + h) * D;
  const float pos = static_cast<float>(positions[t]);
  constexpr int HALF = D / 2;
#pragma unroll
  for (int i = lane; i < HALF; i += 32) {
    const float inv_freq = exp2f(-log2_theta * (static_cast<float>(2 * i) / D));
    float sn, cs;
    sincosf(pos * inv_freq, &sn, &cs);
    if (inverse) sn = -sn;
    const float a = __bfloat162float(src[i]), b = __bfloat162float(src[i + HALF]);
    dst[i] = __float2bfloat16(a * cs - b * sn);
    dst[i + HALF] = __float2bfloat16(b * cs + a * sn);
  }
}

// ---------------------------------------------------------------------------------------------
// KV cache scatter: rows [T, Hkv·D] → cache[slot, Hkv·D]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                             long long k_stride, long long v_stride, __nv_bfloat16* __restrict__ kc,
                                                             __nv_bfloat16* __restrict__ vc, const long long* __restrict__ slots,
                                                             long long T, int row_elems) {
  const int nvec = row_elems / 8;
  const long long total = T * nvec;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const long long t = i / nvec;
    const int c = static_cast<int>(i % nvec) * 8;
    const long long slot = slots[t];
    if (slot < 0 || !dbg::in_bounds(dbg::kKvSlots, slot, 102)) continue;
    *reinterpret_cast<uint4*>(kc + slot * row_elems + c) = *reinterpret_cast<const uint4*>(k + t * k_stride + c);
    *reinterpret_cast<uint4*>(vc + slot * row_elems + c) = *reinterpret_cast<const uint4*>(v + t * v_stride + c);
  }
}

// ---------------------------------------------------------------------------------------------
// AdamW on a flat fp32 shard with a per-element decay mask and a device-side gradient scale; writes the
// updated parameter in bf16 (or fp32) to `param_out`.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                                                    float* __restrict__ v, const float* __restrict__ decay_mask,
                                                    const float* __restrict__ scale_ptr, void* __restrict__ param_out, int out_bf16,
                                                    long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                                                    float bc2) {
  const float scale = scale_ptr ? *scale_ptr : 1.f;
  for (long long i = (blockIdx.x * 256ll + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * 256 * 4) {
    if (i + 4 <= n) {
      float4 g = *reinterpret_cast<const float4*>(grad + i);
      float4 mm = *reinterpret_cast<const float4*>(m + i);
      float4 vv = *reinterpret_cast<const float4*>(v + i);
      float4 p = *reinterpret_cast<const float4*>(master + i);
      float4 dm = decay_mask ? *reinterpret_cast<const float4*>(decay_mask + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      float* gp = reinterpret_cast<float*>(&g);
      float* mp = reinterpret_cast<float*>(&mm);
      float* vp = reinterpret_cast<float*>(&vv);
      float* pp = reinterpret_cast<float*>(&p);
      float* dp = reinterpret_cast<float*>(&dm);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gs = gp[k] * scale;
        mp[k] = b1 * mp[k] + (1.f - b1) * gs;
        vp[k] = b2 * vp[k] + (1.f - b2) * gs * gs;
        const float denom = sqrtf(vp[k] / bc2) + eps;
        pp[k] = pp[k] * (1.f - lr * wd * dp[k]) - lr * (mp[k] / bc1) / denom;
      }
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      *reinterpret_cast<float4*>(master + i) = p;
      if (param_out != nullptr) {
        if (out_bf16) {
          uint2 o;
          __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]);
          __nv_bfloat162 hi = __floats2bfloat162_rn(pp[2], pp[3]);
          o.x = *reinterpret_cast<uint32_t*>(&lo);
          o.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(param_out) + i) = o;
        } else {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(param_out) + i) = p;
        }
      }
    } else {
      for (long long j = i; j < n; ++j) {
        const float gs = grad[j] * scale;
        m[j] = b1 * m[j] + (1.f - b1) * gs;
        v[j] = b2 * v[j] + (1.f - b2) * gs * gs;
        const float denom = sqrtf(v[j] / bc2) + eps;
        const float dm = decay_mask ? decay_mask[j] : 1.f;
        master[j] = master[j] * (1.f - lr * wd * dm) - lr * (m[j] / bc1) / denom;
        if (param_out != nullptr) {
          if (out_bf16) reinterpret_cast<__nv_bfloat16*>(param_out)[j] = __float2bfloat16(master[j]);
          else reinterpret_cast<float*>(param_out)[j] = master[j];
        }
      }
    }
  }
}

static int grid_for(long long work_items, int per_block, int max_blocks = 148 * 8) {
  long long b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

}  // namespace mb

using namespace mb;

MB_DEFINE_BOUNDS_API(mb_elementwise_bounds)

extern "C" int mb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out, float* rstd, long long T,
                              int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  typedef const __nv_bfloat16* cbf;
  typedef __nv_bfloat16* bf;
  cudaError_t e;
  const bool add = residual != nullptr;
  const dim3 wgrid(static_cast<unsigned>((T + 7) / 8));
  // rows of 1024 / 2048 / 4096 elements with 16-byte aligned pointers: one warp per row (T ≥ 64 so that the grid fills the SMs)
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) |
                         reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(res_out)) & 15) == 0;
  if (aligned && T >= 64 && (H == 1024 || H == 2048 || H == 4096)) {
#define MB_RMS_WARP(ADD_, VPL_)                                                                                                    \
  launch_pdl(rmsnorm_fwd_warp_kernel<ADD_, VPL_>, wgrid, dim3(256), 0, s, X, (cbf)residual, (cbf)w, (bf)y, (bf)res_out, rstd, \
             static_cast<long long>(T), eps)
    if (H == 1024) e = add ? MB_RMS_WARP(true, 4) : MB_RMS_WARP(false, 4);
    else if (H == 2048) e = add ? MB_RMS_WARP(true, 8) : MB_RMS_WARP(false, 8);
    else e = add ? MB_RMS_WARP(true, 16) : MB_RMS_WARP(false, 16);
#undef MB_RMS_WARP
    return static_cast<int>(e);
  }
  if (residual != nullptr)
    e = launch_pdl(rmsnorm_fwd_kernel<true>, dim3(static_cast<unsigned>(T)), dim3(256), 0, s, X, (cbf)residual, (cbf)w, (bf)y, (bf)res_out,
                   rstd, H, eps);
  else
    e = launch_pdl(rmsnorm_fwd_kernel<false>, dim3(static_cast<unsigned>(T)), dim3(256), 0, s, X, (cbf) nullptr, (cbf)w, (bf)y,
                   (bf) nullptr, rstd, H, eps);
  return static_cast<int>(e);
}

// dw_partial must hold mb_rmsnorm_bwd_blocks(T) × H floats; dw_out receives the reduced weight gradient.
extern "C" int mb_rmsnorm_bwd_blocks(long long T) { return grid_for(T, 1, 148 * 4); }

extern "C" int mb_rmsnorm_bwd(const void* x, const void* w, const void* dy, const void* dres, const float* rstd, void* dx,
                              float* dw_partial, void* dw_out, int dw_fp32, long long T, int H, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 || H > 8192) return -1;
  const int blocks = mb_rmsnorm_bwd_blocks(T);
  rmsnorm_bwd_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                                            reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(dres),
                                            rstd, reinterpret_cast<__nv_bfloat16*>(dx), dw_partial, static_cast<int>(T), H);
  colsum_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, dw_out, blocks, H, dw_fp32);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_colsum(const float* partial, void* out, int R, int C, int out_fp32, cudaStream_t s) {
  colsum_kernel<<<(C + 255) / 256, 256, 0, s>>>(partial, out, R, C, out_fp32);
  return static_cast<int>(cudaGetLastError());
}

// rows_ptr (optional, device): only the first min(T, *rows_ptr) rows are processed
extern "C" int mb_swiglu_fwd(const void* in, void* out, long long T, int F, const int* rows_ptr, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8) return -1;
  return static_cast<int>(launch_pdl(swiglu_fwd_kernel, dim3(grid_for(T * (F / 8), 256)), dim3(256), 0, s,
                                     reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), T, F, rows_ptr));
}

extern "C" int mb_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, const int* rows_ptr, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                                reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                reinterpret_cast<__nv_bfloat16*>(din), T, F, rows_ptr);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_rope(const void* x, void* y, const int* positions, long long T, int H, int D, long long tok_stride, float theta,
                       int inverse, cudaStream_t s) {
  if (T == 0 || H == 0) return 0;
  const unsigned blocks = static_cast<unsigned>((T * H + 7) / 8);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  if (D == 128) rope_kernel<128><<<blocks, 256, 0, s>>>(X, Y, positions, T, H, tok_stride, log2f(theta), inverse);
  else if (D == 64) rope_kernel<64><<<blocks, 256, 0, s>>>(X, Y, positions, T, H, tok_stride, log2f(theta), inverse);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_qk_norm_rope_fwd(const void* q, const void* k, long long q_stride, long long k_stride, const void* qw, const void* kw,
                                   const int* positions, void* qo, void* ko, float* q_rstd, float* k_rstd, long long T, int Hq, int Hk,
                                   int D, float theta, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  const long long warps = T * (Hq + Hk);
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  const float l2t = log2f(theta);
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto K = reinterpret_cast<const __nv_bfloat16*>(k);
  auto QW = reinterpret_cast<const __nv_bfloat16*>(qw);
  auto KW = reinterpret_cast<const __nv_bfloat16*>(kw);
  auto QO = reinterpret_cast<__nv_bfloat16*>(qo);
  auto KO = reinterpret_cast<__nv_bfloat16*>(ko);
  if (D == 128)
    qk_norm_rope_fwd_kernel<128><<<blocks, 256, 0, s>>>(Q, K, q_stride, k_stride, QW, KW, positions, QO, KO, q_rstd, k_rstd, T, Hq, Hk, l2t, eps);
  else if (D == 64)
    qk_norm_rope_fwd_kernel<64><<<blocks, 256, 0, s>>>(Q, K, q_stride, k_stride, QW, KW, positions, QO, KO, q_rstd, k_rstd, T, Hq, Hk, l2t, eps);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

// Engine (no autograd) form: q/k norm + rotary, and k/v written to the paged cache [slots, Hk, D] in the same launch.
extern "C" int mb_qk_norm_rope_cache(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                     long long v_stride, const void* qw, const void* kw, const int* positions, void* qo, void* ko,
                                     void* kc, void* vc, const long long* slots, long long T, int Hq, int Hk, int D, float theta,
                                     float eps, cudaStream_t s) {
  if (T == 0) return 0;
  const int blocks = static_cast<int>((T * (Hq + 2 * Hk) + 7) / 8);
  const float l2t = log2f(theta);
  typedef const __nv_bfloat16* cbf;
  typedef __nv_bfloat16* bf;
  if (D == 128)
    return static_cast<int>(launch_pdl(qk_norm_rope_cache_kernel<128>, dim3(blocks), dim3(256), 0, s, (cbf)q, (cbf)k, (cbf)v, q_stride, k_stride,
                                       v_stride, (cbf)qw, (cbf)kw, positions, (bf)qo, (bf)ko, (bf)kc, (bf)vc, slots, T, Hq, Hk, l2t, eps));
  if (D == 64)
    return static_cast<int>(launch_pdl(qk_norm_rope_cache_kernel<64>, dim3(blocks), dim3(256), 0, s, (cbf)q, (cbf)k, (cbf)v, q_stride, k_stride,
                                       v_stride, (cbf)qw, (cbf)kw, positions, (bf)qo, (bf)ko, (bf)kc, (bf)vc, slots, T, Hq, Hk, l2t, eps));
  return -1;
}

extern "C" int mb_qk_norm_rope_bwd_blocks(long long T, int Hn) { return grid_for(T * Hn, 8, 148 * 4); }

// One call per tensor (q or k).  dw_partial: blocks × D floats (may be null when w is null).
extern "C" int mb_qk_norm_rope_bwd(const void* x, long long x_stride, const void* w, const float* rstd, const void* dy,
                                   const int* positions, void* dx, long long dx_stride, float* dw_partial, void* dw_out, long long T,
                                   int Hn, int D, float theta, cudaStream_t s) {
  if (T == 0) return 0;
  const int blocks = mb_qk_norm_rope_bwd_blocks(T, Hn);
  const float l2t = log2f(theta);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  if (D == 128)
    qk_norm_rope_bwd_kernel<128><<<blocks, 256, 0, s>>>(X, x_stride, W, rstd, DY, positions, DX, dx_stride, dw_partial, T, Hn, l2t);
  else if (D == 64)
    qk_norm_rope_bwd_kernel<64><<<blocks, 256, 0, s>>>(X, x_stride, W, rstd, DY, positions, DX, dx_stride, dw_partial, T, Hn, l2t);
  else
    return -1;
  if (w != nullptr && dw_out != nullptr) colsum_kernel<<<1, 128, 0, s>>>(dw_partial, dw_out, blocks, D, 0);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_kv_cache_write(const void* k, const void* v, long long k_stride, long long v_stride, void* kc, void* vc,
                                 const long long* slots, long long T, int row_elems, cudaStream_t s) {
  if (T == 0) return 0;
  if (row_elems % 8) return -1;
  kv_cache_write_kernel<<<grid_for(T * (row_elems / 8), 256), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v), k_stride, v_stride,
      reinterpret_cast<__nv_bfloat16*>(kc), reinterpret_cast<__nv_bfloat16*>(vc), slots, T, row_elems);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_adamw(float* master, const float* grad, float* m, float* v, const float* decay_mask, const float* scale_ptr,
                        void* param_out, int out_bf16, long long n, float lr, float b1, float b2, float eps, float wd, int step,
                        cudaStream_t s) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, static_cast<float>(step));
  const float bc2 = 1.f - powf(b2, static_cast<float>(step));
  adamw_kernel<<<grid_for(n, 1024), 256, 0, s>>>(master, grad, m, v, decay_mask, scale_ptr, param_out, out_bf16, n, lr, b1, b2, eps,
                                                wd, bc1, bc2);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward without any allocation (declared in launch.h)
// ---------------------------------------------------------------------------------------------
// Same two kernels as mb_rmsnorm_bwd, but the per-CTA partial weight-gradient rows live in a fixed array in device
// global memory instead of a buffer supplied by the caller.  Nothing is allocated here, by CUDA or by a library.
// The array is one per device and shared by every call on that device:
//   * it keeps whatever the previous call left in it; nothing has to be cleared, because each call first writes every
//     element (rows 0..blocks-1, columns 0..H-1) that its reduction then reads;
//   * two calls that overlap in time on one device (different streams, or threads) write the same rows and race:
//     the caller orders them.
// Limit: H ≤ MB_RMSNORM_BWD_STATIC_MAX_H; larger H is refused with MB_ERR_STATIC_SCRATCH_TOO_SMALL.
static constexpr int kStaticBwdMaxBlocks = 148 * 4;   // the largest grid mb_rmsnorm_bwd_blocks() returns
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[static_cast<size_t>(kStaticBwdMaxBlocks) * MB_RMSNORM_BWD_STATIC_MAX_H];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_scratch_addr[kMaxDevices];   // device address of the array, looked up once per device
}  // namespace

extern "C" const char* mb_rmsnorm_bwd_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "mb_rmsnorm_bwd_static: H must be a multiple of 8";
    case MB_ERR_STATIC_SCRATCH_TOO_SMALL:
      return "mb_rmsnorm_bwd_static: H exceeds MB_RMSNORM_BWD_STATIC_MAX_H (4096), the width the fixed scratch array holds; "
             "use mb_rmsnorm_bwd with a caller-provided buffer";
    case MB_ERR_STATIC_SCRATCH_SETUP: return "mb_rmsnorm_bwd_static: could not resolve the scratch array's device address";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "mb_rmsnorm_bwd_static: unknown error";
  }
}

extern "C" int mb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const void* dres, const float* rstd, void* dx,
                                     void* dw_out, int dw_fp32, long long T, int H, cudaStream_t s) {
  if (H % 8) return -1;
  if (H > MB_RMSNORM_BWD_STATIC_MAX_H) return MB_ERR_STATIC_SCRATCH_TOO_SMALL;
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return static_cast<int>(rc);
  if (dev < 0 || dev >= kMaxDevices) return MB_ERR_STATIC_SCRATCH_SETUP;
  float* scratch = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (scratch == nullptr) {
    // First call on this device: resolve the symbol (this may load the module, so it belongs before any stream capture).
    void* p = nullptr;
    rc = cudaGetSymbolAddress(&p, g_rmsnorm_bwd_scratch);
    if (rc != cudaSuccess) return static_cast<int>(rc);
    if (p == nullptr) return MB_ERR_STATIC_SCRATCH_SETUP;
    scratch = static_cast<float*>(p);
    __atomic_store_n(&g_static_scratch_addr[dev], scratch, __ATOMIC_RELEASE);   // racing first calls store the same value
  }
  if (T == 0) return 0;
  const int blocks = mb_rmsnorm_bwd_blocks(T);
  if (blocks > kStaticBwdMaxBlocks) return MB_ERR_STATIC_SCRATCH_TOO_SMALL;
  mb::rmsnorm_bwd_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                                                reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(dres),
                                                rstd, reinterpret_cast<__nv_bfloat16*>(dx), scratch, static_cast<int>(T), H);
  mb::colsum_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, dw_out, blocks, H, dw_fp32);
  return static_cast<int>(cudaGetLastError());
}
