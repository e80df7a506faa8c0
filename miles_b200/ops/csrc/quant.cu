// Quantisation kernels.
//   mxfp8_quant      1×32 blocks, e4m3 payload, e8m0 (power-of-two) scales — training / weight-sync format
//   fp8_block_quant  128×128 blocks, e4m3 payload, fp32 scale_inv — inference weight format
//   int4_fake_quant  quantise→dequantise to int4 per [bm, bn] block, symmetric (/7) or asymmetric (/15 + zero point)
//   nvfp4_qdq        quantise→dequantise to e2m1 with e4m3 1×16 block scales and an fp32 tensor scale
//   block_fake_quant quantise→dequantise in one pass: 1×32 blocks with a power-of-two scale and an e4m3 or e2m1 payload
//                    (MXFP8 / MXFP4 style), or 1×16 blocks with an e4m3 scale and an e2m1 payload (compressed-KV style)
//   absmax           fp32 max |x| of a tensor (tensor scale for nvfp4)
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(h[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// ---- MXFP8: one thread per 32-element block -------------------------------------------------------
__global__ void __launch_bounds__(256) mxfp8_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ scales,
                                                          long long nblocks) {
  const long long b = blockIdx.x * 256ll + threadIdx.x;
  if (b >= nblocks) return;
  float v[32];
#pragma unroll
  for (int i = 0; i < 4; ++i) ld8(x + b * 32 + i * 8, *reinterpret_cast<float(*)[8]>(&v[i * 8]));
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  // biased exponent e with amax / 2^(e−127) ≤ 448: e − 127 = ceil(log2(amax / 448))
  const float ratio = fmaxf(amax * (1.f / 448.f), 1.17549435e-38f);
  const uint32_t bits = __float_as_uint(ratio);
  int e = static_cast<int>((bits >> 23) & 0xff);
  if (bits & 0x7fffff) e += 1;
  e = min(max(e, 0), 254);
  const float inv_scale = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);  // 2^(127 − e)
  scales[b] = static_cast<uint8_t>(e);
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    out[i] = e4m3x4(v[4 * i] * inv_scale, v[4 * i + 1] * inv_scale, v[4 * i + 2] * inv_scale, v[4 * i + 3] * inv_scale);
  uint4* dst = reinterpret_cast<uint4*>(q + b * 32);
  dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
  dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
}

// ---- block fake quantisation: 8 elements per lane, 4 lanes per 32-block (2 per 16-block) -------------------------------
// MODE 0: 32-block, power-of-two scale, e4m3 payload.  MODE 1: 32-block, power-of-two scale, e2m1 payload.
// MODE 2: 16-block, e4m3 scale clamped to [2^-9, 448], e2m1 payload.
__device__ __forceinline__ float e2m1_round(float v) {          // v already clamped to [−6, 6]; ties to even, as rint on the grid
  const float mag = fabsf(v);
  const float step = mag < 2.f ? 0.5f : (mag < 4.f ? 1.f : 2.f);
  const float q = rintf(mag * (mag < 2.f ? 2.f : (mag < 4.f ? 1.f : 0.5f))) * step;    // steps are powers of two: exact
  return copysignf(q, v);
}
__device__ __forceinline__ float e4m3_round(float v) {
  const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}
template <int MODE>
__global__ void __launch_bounds__(256) block_fake_quant_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n8) {
  // two 16-byte groups per thread, 256 groups apart: both loads are in flight before either is used (the kernel is bound by
  // load latency at one group per thread: ~10 stalled warps per issue on the long scoreboard)
  constexpr int U = 2;
  const long long base = blockIdx.x * (256ll * U) + threadIdx.x;
  float v[U][8];
  bool live[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long long i = base + u * 256;
    live[u] = i < n8;
#pragma unroll
    for (int k = 0; k < 8; ++k) v[u][k] = 0.f;
    if (live[u]) ld8(x + i * 8, v[u]);
  }
  constexpr float FMAX = MODE == 0 ? 448.f : 6.f;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[u][k]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (MODE != 2) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale, inv_scale = 0.f;
    if (MODE == 2) {
      scale = e4m3_round(fminf(fmaxf(amax * (1.f / 6.f), 0.001953125f), 448.f));
    } else {
      const float floor_ = MODE == 0 ? 1e-4f : 6.f * 1.17549435e-38f;
      const uint32_t bits = __float_as_uint(fmaxf(amax, floor_) * (1.f / FMAX));
      int e = static_cast<int>((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffff) ? 1 : 0);     // ceil to a power of two
      scale = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
      inv_scale = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);       // the reciprocal of a power of two is exact
    }
    if (!live[u]) continue;
    __nv_bfloat162 out[4];
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      float a = MODE == 2 ? __fdiv_rn(v[u][k], scale) : v[u][k] * inv_scale, b = MODE == 2 ? __fdiv_rn(v[u][k + 1], scale) : v[u][k + 1] * inv_scale;
      a = fminf(fmaxf(a, -FMAX), FMAX);
      b = fminf(fmaxf(b, -FMAX), FMAX);
      a = (MODE == 0 ? e4m3_round(a) : e2m1_round(a)) * scale;
      b = (MODE == 0 ? e4m3_round(b) : e2m1_round(b)) * scale;
      out[k / 2] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<uint4*>(y + (base + u * 256) * 8) = *reinterpret_cast<const uint4*>(out);
  }
}

// ---- FP8 128×128 blocks: one CTA per block ----------------------------------------------------------
__global__ void __launch_bounds__(256) fp8_block_quant_kernel(const bf16* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ scale_inv,
                                                              int M, int N) {
  __shared__ float red[8];
  const int bm = blockIdx.y, bn = blockIdx.x;
  const int r0 = bm * 128, c0 = bn * 128;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 16; i += 256) {   // 16 chunks of 8 per row
    const int r = r0 + i / 16, c = c0 + (i % 16) * 8;
    if (r < M && c < N) {
      if (c + 8 <= N) {
        float f[8];
        ld8(w + static_cast<long long>(r) * N + c, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
      } else {
        for (int k = 0; c + k < N; ++k) amax = fmaxf(amax, fabsf(__bfloat162float(w[static_cast<long long>(r) * N + c + k])));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  amax = fmaxf(amax, 1e-12f);
  const float sinv = amax / 448.f;
  const float s = 448.f / amax;
  if (threadIdx.x == 0) scale_inv[bm * gridDim.x + bn] = sinv;
  for (int i = threadIdx.x; i < 128 * 16; i += 256) {
    const int r = r0 + i / 16, c = c0 + (i % 16) * 8;
    if (r < M && c < N) {
      if (c + 8 <= N) {
        float f[8];
        ld8(w + static_cast<long long>(r) * N + c, f);
        uint2 o;
        o.x = e4m3x4(f[0] * s, f[1] * s, f[2] * s, f[3] * s);
        o.y = e4m3x4(f[4] * s, f[5] * s, f[6] * s, f[7] * s);
        *reinterpret_cast<uint2*>(q + static_cast<long long>(r) * N + c) = o;
      } else {
        for (int k = 0; c + k < N; ++k) {
          const float f = __bfloat162float(w[static_cast<long long>(r) * N + c + k]) * s;
          q[static_cast<long long>(r) * N + c + k] =
              static_cast<uint8_t>(__nv_cvt_float2_to_fp8x2(make_float2(f, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xff);
        }
      }
    }
  }
}

// ---- INT4 fake quant: one warp per [bm, bn] block -------------------------------------------------------
__global__ void __launch_bounds__(256) int4_fake_quant_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, float* __restrict__ scales,
                                                              int M, int N, int bm, int bn, int symmetric) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int nb_n = N / bn, nb_m = M / bm;
  if (wid >= static_cast<long long>(nb_m) * nb_n) return;
  const int br = static_cast<int>(wid / nb_n), bc = static_cast<int>(wid % nb_n);
  const int elems = bm * bn;
  float mx = -INFINITY, mn = INFINITY;
  for (int i = lane; i < elems; i += 32) {
    const float v = __bfloat162float(x[static_cast<long long>(br * bm + i / bn) * N + bc * bn + i % bn]);
    mx = fmaxf(mx, v);
    mn = fminf(mn, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  float scale, zp = 0.f;
  if (symmetric) {
    scale = fmaxf(fmaxf(fabsf(mx), fabsf(mn)) / 7.f, 1e-10f);
  } else {
    scale = fmaxf((mx - mn) / 15.f, 1e-10f);
    zp = rintf(-mn / scale);
  }
  if (lane == 0 && scales != nullptr) scales[wid] = scale;
  for (int i = lane; i < elems; i += 32) {
    const long long off = static_cast<long long>(br * bm + i / bn) * N + bc * bn + i % bn;
    const float v = __bfloat162float(x[off]);
    float o;
    if (symmetric) {
      o = fminf(fmaxf(rintf(v / scale), -8.f), 7.f) * scale;
    } else {
      o = (fminf(fmaxf(rintf(v / scale) + zp, 0.f), 15.f) - zp) * scale;
    }
    y[off] = __float2bfloat16(o);
  }
}

// ---- NVFP4 quantise→dequantise ---------------------------------------------------------------------------
// Two adjacent lanes share one 1×16 block: each loads and stores 16 bytes (every warp access is one contiguous 512-byte
// run), the block maximum and the candidates' errors meet through one shuffle.  FOS ("four over six"): the block is
// quantised twice, with its maximum mapped to 6 and to 4 (finer steps when the values crowd the upper half of the e2m1
// grid), and the candidate with the smaller squared error is kept.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .b8 t;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n\t"
      "cvt.u32.u8 %0, t;\n\t}\n"
      : "=r"(r)
      : "f"(lo), "f"(hi));
  return r;  // low nibble = lo, high nibble = hi
}
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t code) {
  uint32_t h2;
  asm volatile(
      "{\n\t.reg .b8 t;\n\t"
      "cvt.u8.u32 t, %1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, t;\n\t}\n"
      : "=r"(h2)
      : "r"(code));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

__device__ __forceinline__ float nvfp4_candidate(const float (&v)[8], float amax, float gscale, float target, float (&o)[8]) {
  const float sb_f = fminf(amax / target * gscale, 448.f);
  const __nv_fp8_storage_t sb8 = __nv_cvt_float_to_fp8(sb_f, __NV_SATFINITE, __NV_E4M3);
  const float sb = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb8, __NV_E4M3)));
  const float dec = sb / gscale;
  const float enc = dec > 0.f ? 1.f / dec : 0.f;
  float err = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    const float2 q = e2m1x2_to_float2(cvt_e2m1x2(v[i] * enc, v[i + 1] * enc));
    o[i] = q.x * dec;
    o[i + 1] = q.y * dec;
    err += (o[i] - v[i]) * (o[i] - v[i]) + (o[i + 1] - v[i + 1]) * (o[i + 1] - v[i + 1]);
  }
  return err;
}

template <bool FOS>
__global__ void __launch_bounds__(256) nvfp4_qdq_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ global_amax,
                                                        long long npieces) {   // pieces of 8 elements; even, so partner lanes live or die together
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  const bool live = i < npieces;
  float v[8];
  if (live) {
    ld8(x + i * 8, v);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  const float gscale = (448.f * 6.f) / fmaxf(__ldg(global_amax), 1e-12f);
  float o[8];
  float e6 = nvfp4_candidate(v, amax, gscale, 6.f, o);
  if (FOS) {
    float o4[8];
    float e4 = nvfp4_candidate(v, amax, gscale, 4.f, o4);
    e6 += __shfl_xor_sync(0xffffffffu, e6, 1);
    e4 += __shfl_xor_sync(0xffffffffu, e4, 1);
    if (e4 < e6) {
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = o4[k];
    }
  }
  if (!live) return;
  uint4 w;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(o[2 * k], o[2 * k + 1]);
  *reinterpret_cast<uint4*>(y + i * 8) = w;
}

__global__ void __launch_bounds__(256) absmax_kernel(const bf16* __restrict__ x, float* __restrict__ out, long long n) {
  float m = 0.f;
  for (long long i = (blockIdx.x * 256ll + threadIdx.x) * 8; i + 8 <= n; i += static_cast<long long>(gridDim.x) * 256 * 8) {
    float f[8];
    ld8(x + i, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(f[k]));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n - (n % 8); i < n; ++i) m = fmaxf(m, fabsf(__bfloat162float(x[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));  // valid for non-negative floats
}

}  // namespace mb

using namespace mb;

extern "C" int mb_mxfp8_quant(const void* x, void* q, void* scales, long long numel, cudaStream_t s) {
  if (numel == 0) return 0;
  if (numel % 32) return -1;
  const long long nb = numel / 32;
  mxfp8_quant_kernel<<<static_cast<unsigned>((nb + 255) / 256), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<uint8_t*>(q),
                                                                            reinterpret_cast<uint8_t*>(scales), nb);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_fp8_block_quant(const void* w, void* q, float* scale_inv, int M, int N, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + 127) / 128, (M + 127) / 128);
  fp8_block_quant_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(w), reinterpret_cast<uint8_t*>(q), scale_inv, M, N);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_int4_fake_quant(const void* x, void* y, float* scales, int M, int N, int bm, int bn, int symmetric, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  if (M % bm || N % bn) return -1;
  const long long warps = static_cast<long long>(M / bm) * (N / bn);
  int4_fake_quant_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(y),
                                                                               scales, M, N, bm, bn, symmetric);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_nvfp4_qdq(const void* x, void* y, const float* global_amax, long long numel, int four_over_six, cudaStream_t s) {
  if (numel == 0) return 0;
  if (numel % 16) return -1;
  const long long np = numel / 8;
  const unsigned grid = static_cast<unsigned>((np + 255) / 256);
  if (four_over_six)
    nvfp4_qdq_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(y), global_amax, np);
  else
    nvfp4_qdq_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(y), global_amax, np);
  return static_cast<int>(cudaGetLastError());
}

// mode 0: MXFP8-style, 1: MXFP4-style, 2: compressed-KV style (see block_fake_quant_kernel); numel a multiple of 32 (16 for mode 2)
extern "C" int mb_block_fake_quant(const void* x, void* y, long long numel, int mode, cudaStream_t s) {
  if (numel == 0) return 0;
  if (mode < 0 || mode > 2 || numel % (mode == 2 ? 16 : 32)) return -1;
  const long long n8 = numel / 8;
  const unsigned grid = static_cast<unsigned>((n8 + 511) / 512);     // two groups of 8 elements per thread
  const bf16* X = reinterpret_cast<const bf16*>(x);
  bf16* Y = reinterpret_cast<bf16*>(y);
  if (mode == 0) block_fake_quant_kernel<0><<<grid, 256, 0, s>>>(X, Y, n8);
  else if (mode == 1) block_fake_quant_kernel<1><<<grid, 256, 0, s>>>(X, Y, n8);
  else block_fake_quant_kernel<2><<<grid, 256, 0, s>>>(X, Y, n8);
  return static_cast<int>(cudaGetLastError());
}

// out must be zero-initialised by the caller
extern "C" int mb_absmax(const void* x, float* out, long long numel, cudaStream_t s) {
  if (numel == 0) return 0;
  long long blocks = (numel / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  absmax_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), out, numel);
  return static_cast<int>(cudaGetLastError());
}
