// Quantisation kernels.
//   mxfp8_quant      1×32 blocks, e4m3 payload, e8m0 (power-of-two) scales — training / weight-sync format
//   fp8_block_quant  128×128 blocks, e4m3 payload, fp32 scale_inv — inference weight format
//   int4_fake_quant  quantise→dequantise to int4 per [bm, bn] block, symmetric (/7) or asymmetric (/15 + zero point)
//   nvfp4_qdq        quantise→dequantise to e2m1 with e4m3 1×16 block scales and an fp32 tensor scale
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

// ---- NVFP4 quantise→dequantise: one thread per 16-element block -----------------------------------------
__device__ __forceinline__ float e2m1_value(uint32_t code) {   // 4-bit sign|exp(2)|mant(1)
  const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = mag[code & 7];
  return (code & 8) ? -v : v;
}
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

__global__ void __launch_bounds__(256) nvfp4_qdq_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ global_amax,
                                                        long long nblocks) {
  const long long b = blockIdx.x * 256ll + threadIdx.x;
  if (b >= nblocks) return;
  float v[16];
  ld8(x + b * 16, *reinterpret_cast<float(*)[8]>(&v[0]));
  ld8(x + b * 16 + 8, *reinterpret_cast<float(*)[8]>(&v[8]));
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float gscale = (448.f * 6.f) / fmaxf(*global_amax, 1e-12f);
  const float sb_f = fminf(amax / 6.f * gscale, 448.f);
  const __nv_fp8_storage_t sb8 = __nv_cvt_float_to_fp8(sb_f, __NV_SATFINITE, __NV_E4M3);
  const float sb = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb8, __NV_E4M3)));
  const float dec = sb / gscale;
  const float enc = dec > 0.f ? 1.f / dec : 0.f;
  float o[16];
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const uint32_t code = cvt_e2m1x2(v[i] * enc, v[i + 1] * enc);
    o[i] = e2m1_value(code & 0xf) * dec;
    o[i + 1] = e2m1_value((code >> 4) & 0xf) * dec;
  }
  uint4 w0, w1;
  __nv_bfloat162* p0 = reinterpret_cast<__nv_bfloat162*>(&w0);
  __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&w1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    p0[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
    p1[i] = __floats2bfloat162_rn(o[8 + 2 * i], o[8 + 2 * i + 1]);
  }
  *reinterpret_cast<uint4*>(y + b * 16) = w0;
  *reinterpret_cast<uint4*>(y + b * 16 + 8) = w1;
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

extern "C" int mb_nvfp4_qdq(const void* x, void* y, const float* global_amax, long long numel, cudaStream_t s) {
  if (numel == 0) return 0;
  if (numel % 16) return -1;
  const long long nb = numel / 16;
  nvfp4_qdq_kernel<<<static_cast<unsigned>((nb + 255) / 256), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<bf16*>(y),
                                                                          global_amax, nb);
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
