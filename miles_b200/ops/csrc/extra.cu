// Row-wise / elementwise kernels of the non-Qwen model families and of the quantisation tools.
//   grouped_rmsnorm      per (token, stream) RMS norm over C channels, scale (1 + w), fp32 out        [T, n·C]
//   short_conv           residual causal depthwise conv of width W over packed sequences               [T, D]
//   mhc_mix              out[j] = h_post[j]·x + Σ_i h_res[i][j]·residual[i]   (n residual streams)     [T, n·d]
//   mhc_aggregate        out = Σ_i pre[i]·x[i]  in fp32                                                [T, d]
//   hc_combine           out[c] = residual[c] + h_post[c]·y                                            [T, n·C]
//   act_quant_1x128      per-row 128-wide FP8 e4m3 blocks, fp32 (optionally power-of-two) scales; or quantise→dequantise
//   fp8_block_dequant    128×128-block e4m3 × fp32 scale_inv → bf16;  mxfp8_dequant  1×32 e4m3 × 2^(e−127) → bf16
//   gather_rows_host     rows of a table in PINNED HOST memory gathered straight into device memory (zero-copy reads)
// All are bandwidth-bound: 16-byte accesses, one pass, fp32 math.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// one warp per (token, stream); x bf16 or fp32
template <typename TIn>
__global__ void __launch_bounds__(256) grouped_rmsnorm_kernel(const TIn* __restrict__ x, const float* __restrict__ w,
                                                              float* __restrict__ out, float* __restrict__ rstd, long long rows,
                                                              int n, int C, float eps) {
  const long long r = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int c = static_cast<int>(r % n);
  const TIn* xr = x + r * C;
  float ss = 0.f;
  for (int i = lane; i < C; i += 32) {
    const float v = static_cast<float>(xr[i]);
    ss += v * v;
  }
  const float rs = rsqrtf(warp_sum_f(ss) / C + eps);
  if (lane == 0 && rstd != nullptr) rstd[r] = rs;
  for (int i = lane; i < C; i += 32) out[r * C + i] = static_cast<float>(xr[i]) * rs * (1.f + w[c * C + i]);
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                         const int* __restrict__ bos, T* __restrict__ y, long long Tn, int D, int W) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= Tn * D) return;
  const long long t = i / D;
  const int d = static_cast<int>(i % D);
  const long long b = bos[t];
  const float cur = static_cast<float>(x[i]);
  float acc = cur;                                        // residual
  for (int iw = 0; iw < W; ++iw) {
    const long long s = t - (W - 1) + iw;
    if (s >= b) acc += static_cast<float>(x[s * D + d]) * w[d * W + iw];
  }
  y[i] = static_cast<T>(acc);
}

template <typename T>
__global__ void __launch_bounds__(256) mhc_mix_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ h_res,
                                                      const float* __restrict__ h_post, T* __restrict__ out, long long Tn, int n, int d) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= Tn * n * d) return;
  const long long t = i / (static_cast<long long>(n) * d);
  const int j = static_cast<int>((i / d) % n), k = static_cast<int>(i % d);
  float acc = h_post[t * n + j] * static_cast<float>(x[t * d + k]);
  for (int s = 0; s < n; ++s) acc += h_res[(t * n + s) * n + j] * static_cast<float>(res[(t * n + s) * d + k]);
  out[i] = static_cast<T>(acc);
}

template <typename T>
__global__ void __launch_bounds__(256) mhc_aggregate_kernel(const T* __restrict__ x, const float* __restrict__ pre, float* __restrict__ out,
                                                            long long Tn, int n, int d) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= Tn * d) return;
  const long long t = i / d;
  const int k = static_cast<int>(i % d);
  float acc = 0.f;
  for (int s = 0; s < n; ++s) acc += pre[t * n + s] * static_cast<float>(x[(t * n + s) * d + k]);
  out[i] = acc;
}

template <typename T>
__global__ void __launch_bounds__(256) hc_combine_kernel(const T* __restrict__ res, const T* __restrict__ y, const float* __restrict__ h_post,
                                                         T* __restrict__ out, long long Tn, int n, int C) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= Tn * n * C) return;
  const long long t = i / (static_cast<long long>(n) * C);
  const int c = static_cast<int>((i / C) % n), k = static_cast<int>(i % C);
  out[i] = static_cast<T>(static_cast<float>(res[i]) + h_post[t * n + c] * static_cast<float>(y[t * C + k]));
}

// one warp per (row, 128-column block): 4 elements per lane
__global__ void __launch_bounds__(256) act_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, bf16* __restrict__ qdq,
                                                        float* __restrict__ scales, long long M, int N, int round_scale) {
  const int nb = N / 128;
  const long long wid = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= M * nb) return;
  const long long row = wid / nb;
  const int blk = static_cast<int>(wid % nb);
  const bf16* src = x + row * N + blk * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(warp_max_f(amax), 1e-4f);
  float s = amax * (1.f / 448.f);
  if (round_scale) {                                     // smallest power of two ≥ s
    const uint32_t bits = __float_as_uint(s);
    const uint32_t e = ((bits >> 23) & 0xff) + ((bits & 0x7fffff) ? 1 : 0);
    s = __uint_as_float(e << 23);
  }
  const float inv = 1.f / s;
  const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
  if (lane == 0) scales[row * nb + blk] = s;
  if (q != nullptr)
    *reinterpret_cast<uint32_t*>(q + row * N + blk * 128 + lane * 4) = static_cast<uint32_t>(p0) | (static_cast<uint32_t>(p1) << 16);
  if (qdq != nullptr) {
    const __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2(p0, __NV_E4M3), r1 = __nv_cvt_fp8x2_to_halfraw2(p1, __NV_E4M3);
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&r0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&r1));
    __nv_bfloat162 o[2] = {__floats2bfloat162_rn(f0.x * s, f0.y * s), __floats2bfloat162_rn(f1.x * s, f1.y * s)};
    *reinterpret_cast<uint2*>(qdq + row * N + blk * 128 + lane * 4) = *reinterpret_cast<const uint2*>(o);
  }
}

// block_n == 0: per-128×128-block fp32 scale_inv [ceil(M/128), ceil(N/128)]; else e8m0 scales per 1×32 block [M, N/32]
__global__ void __launch_bounds__(256) fp8_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale_inv,
                                                          const uint8_t* __restrict__ e8m0, bf16* __restrict__ out, long long M, int N) {
  const long long i = (blockIdx.x * 256ll + threadIdx.x) * 4;
  if (i >= M * N) return;
  const long long r = i / N;
  const int c = static_cast<int>(i % N);                 // N % 4 == 0: the four elements share a row and a block
  float s;
  if (e8m0 != nullptr) {
    const uint32_t e = e8m0[r * (N / 32) + c / 32];
    s = __uint_as_float((e ? e : 1u) << 23);
  } else {
    s = scale_inv[(r / 128) * ((N + 127) / 128) + c / 128];
  }
  const uint32_t w = *reinterpret_cast<const uint32_t*>(q + i);
  const __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xffff), __NV_E4M3);
  const __half2_raw r1 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
  const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&r0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&r1));
  __nv_bfloat162 o[2] = {__floats2bfloat162_rn(f0.x * s, f0.y * s), __floats2bfloat162_rn(f1.x * s, f1.y * s)};
  *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<const uint2*>(o);
}

// table: device-visible address of pinned host memory [rows, row_bytes]; one warp per output row, 16-byte chunks
__global__ void __launch_bounds__(256) gather_rows_host_kernel(const uint4* __restrict__ table, const long long* __restrict__ ids,
                                                               uint4* __restrict__ out, long long n, int vec_per_row, long long table_rows) {
  const long long r = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= n) return;
  const long long id = ids[r];
  const bool ok = id >= 0 && id < table_rows;
  for (int v = lane; v < vec_per_row; v += 32)
    out[r * vec_per_row + v] = ok ? table[id * vec_per_row + v] : make_uint4(0, 0, 0, 0);
}

inline unsigned blocks_of(long long items) { return static_cast<unsigned>((items + 255) / 256); }

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" int mb_grouped_rmsnorm(const void* x, int x_fp32, const float* w, float* out, float* rstd, long long T, int n, int C, float eps,
                                  cudaStream_t s) {
  const long long rows = T * n;
  if (rows == 0) return 0;
  if (x_fp32) grouped_rmsnorm_kernel<float><<<blocks_of(rows * 32), 256, 0, s>>>(static_cast<const float*>(x), w, out, rstd, rows, n, C, eps);
  else grouped_rmsnorm_kernel<bf16><<<blocks_of(rows * 32), 256, 0, s>>>(static_cast<const bf16*>(x), w, out, rstd, rows, n, C, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_short_conv(const void* x, int fp32, const float* w, const int* bos, void* y, long long T, int D, int W, cudaStream_t s) {
  if (T == 0) return 0;
  if (fp32) short_conv_kernel<float><<<blocks_of(T * D), 256, 0, s>>>(static_cast<const float*>(x), w, bos, static_cast<float*>(y), T, D, W);
  else short_conv_kernel<bf16><<<blocks_of(T * D), 256, 0, s>>>(static_cast<const bf16*>(x), w, bos, static_cast<bf16*>(y), T, D, W);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_mhc_mix(const void* x, const void* res, const float* h_res, const float* h_post, void* out, int fp32, long long T, int n,
                          int d, cudaStream_t s) {
  if (T == 0) return 0;
  if (fp32) mhc_mix_kernel<float><<<blocks_of(T * n * d), 256, 0, s>>>(static_cast<const float*>(x), static_cast<const float*>(res), h_res, h_post, static_cast<float*>(out), T, n, d);
  else mhc_mix_kernel<bf16><<<blocks_of(T * n * d), 256, 0, s>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(res), h_res, h_post, static_cast<bf16*>(out), T, n, d);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_mhc_aggregate(const void* x, int fp32, const float* pre, float* out, long long T, int n, int d, cudaStream_t s) {
  if (T == 0) return 0;
  if (fp32) mhc_aggregate_kernel<float><<<blocks_of(T * d), 256, 0, s>>>(static_cast<const float*>(x), pre, out, T, n, d);
  else mhc_aggregate_kernel<bf16><<<blocks_of(T * d), 256, 0, s>>>(static_cast<const bf16*>(x), pre, out, T, n, d);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_hc_combine(const void* res, const void* y, const float* h_post, void* out, int fp32, long long T, int n, int C, cudaStream_t s) {
  if (T == 0) return 0;
  if (fp32) hc_combine_kernel<float><<<blocks_of(T * n * C), 256, 0, s>>>(static_cast<const float*>(res), static_cast<const float*>(y), h_post, static_cast<float*>(out), T, n, C);
  else hc_combine_kernel<bf16><<<blocks_of(T * n * C), 256, 0, s>>>(static_cast<const bf16*>(res), static_cast<const bf16*>(y), h_post, static_cast<bf16*>(out), T, n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_act_quant_1x128(const void* x, void* q, void* qdq, float* scales, long long M, int N, int round_scale, cudaStream_t s) {
  if (M == 0) return 0;
  if (N % 128) return -1;
  act_quant_kernel<<<blocks_of(M * (N / 128) * 32), 256, 0, s>>>(static_cast<const bf16*>(x), static_cast<uint8_t*>(q), static_cast<bf16*>(qdq), scales, M, N, round_scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_fp8_dequant(const void* q, const float* scale_inv, const void* e8m0, void* out, long long M, int N, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  if (N % 4 || (e8m0 != nullptr && N % 32)) return -1;
  fp8_dequant_kernel<<<blocks_of(M * N / 4), 256, 0, s>>>(static_cast<const uint8_t*>(q), scale_inv, static_cast<const uint8_t*>(e8m0), static_cast<bf16*>(out), M, N);
  return static_cast<int>(cudaGetLastError());
}

// `table_dev` is the device-side alias of a pinned host allocation (cudaHostGetDevicePointer); row_bytes % 16 == 0
extern "C" int mb_gather_rows_host(const void* table_dev, const long long* ids, void* out, long long n, int row_bytes, long long table_rows,
                                   cudaStream_t s) {
  if (n == 0) return 0;
  if (row_bytes % 16) return -1;
  gather_rows_host_kernel<<<blocks_of(n * 32), 256, 0, s>>>(static_cast<const uint4*>(table_dev), ids, static_cast<uint4*>(out), n, row_bytes / 16, table_rows);
  return static_cast<int>(cudaGetLastError());
}
