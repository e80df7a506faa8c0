// Weight synchronisation trainer → engine as ONE launch per bucket.
//
// A bucket is a device table of tensors {src, dst, elements, scale_dst}.  The kernels walk all tensors of the bucket in
// one persistent grid (chunks found by binary search in a prefix array), so a 48-layer model syncs in a handful of
// launches instead of one copy per parameter.  `dst` may be any address this GPU can store to: the engine's buffers on
// the same GPU, or a peer GPU's buffers mapped through CUDA IPC (plain stores over NVLink).
//   multi_copy        bf16/any dtype byte copy (16-byte vectors, byte tail)
//   multi_mxfp8       bf16 → e4m3 payload + e8m0 scales per 1×32 block, quantised on the way (engine serves MXFP8)
//   multi_qdq_mxfp8   bf16 → MXFP8 → bf16 (engine keeps bf16 buffers but sees the values the quantised model would)
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kChunkBytes = 16384;          // per work item for copies
constexpr int kChunkBlocks = 256;           // 1×32 blocks per work item for quantisation (one per thread)

struct Desc {
  long long src, dst, n, aux;               // n: bytes (copy) or elements (quant); aux: scale destination
};

__device__ __forceinline__ int find_desc(const long long* __restrict__ prefix, int n, long long chunk) {
  int lo = 0, hi = n;                        // prefix[lo] <= chunk < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= chunk) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(256) multi_copy_kernel(const Desc* __restrict__ table, const long long* __restrict__ prefix, int n) {
  const long long total = prefix[n];
  for (long long c = blockIdx.x; c < total; c += gridDim.x) {
    const int d = find_desc(prefix, n, c);
    const Desc t = table[d];
    const long long off = (c - prefix[d]) * kChunkBytes;
    const long long len = min(static_cast<long long>(kChunkBytes), t.n - off);
    const char* src = reinterpret_cast<const char*>(t.src) + off;
    char* dst = reinterpret_cast<char*>(t.dst) + off;
    if (((t.src | t.dst) & 15) == 0) {
      const int nv = static_cast<int>(len >> 4);
      for (int i = threadIdx.x; i < nv; i += 256) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
      for (int i = (nv << 4) + threadIdx.x; i < len; i += 256) dst[i] = src[i];
    } else {
      for (int i = threadIdx.x; i < len; i += 256) dst[i] = src[i];
    }
  }
}

__device__ __forceinline__ void ld8(const bf16* p, float* f) {
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

// biased e8m0 exponent e with amax / 2^(e−127) ≤ 448
__device__ __forceinline__ int e8m0_for(float amax) {
  const float ratio = fmaxf(amax * (1.f / 448.f), 1.17549435e-38f);
  const uint32_t bits = __float_as_uint(ratio);
  int e = static_cast<int>((bits >> 23) & 0xff);
  if (bits & 0x7fffff) e += 1;
  return min(max(e, 0), 254);
}

template <bool QDQ>
__global__ void __launch_bounds__(256) multi_mxfp8_kernel(const Desc* __restrict__ table, const long long* __restrict__ prefix, int n) {
  const long long total = prefix[n];
  for (long long c = blockIdx.x; c < total; c += gridDim.x) {
    const int d = find_desc(prefix, n, c);
    const Desc t = table[d];
    const long long b = (c - prefix[d]) * kChunkBlocks + threadIdx.x;   // 1×32 block of this tensor
    if (b * 32 >= t.n) continue;
    const bf16* x = reinterpret_cast<const bf16*>(t.src) + b * 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) ld8(x + i * 8, v + i * 8);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const int e = e8m0_for(amax);
    const float inv_scale = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);   // 2^(127 − e)
    uint32_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      q[i] = e4m3x4(v[4 * i] * inv_scale, v[4 * i + 1] * inv_scale, v[4 * i + 2] * inv_scale, v[4 * i + 3] * inv_scale);
    if (!QDQ) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(t.dst) + b * 32);
      dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
      dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
      reinterpret_cast<uint8_t*>(t.aux)[b] = static_cast<uint8_t>(e);
    } else {
      const float scale = __uint_as_float(static_cast<uint32_t>(max(e, 1)) << 23);   // 2^(e − 127)
      bf16* dst = reinterpret_cast<bf16*>(t.dst) + b * 32;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t w = q[2 * i + (k >> 1)];
          const __nv_fp8x2_storage_t pair = static_cast<__nv_fp8x2_storage_t>((k & 1) ? (w >> 16) : (w & 0xffff));
          const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
          o[k] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
        }
        reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(o);
      }
    }
  }
}

// ---- resharding copy: rectangles between tensors of different row pitch ---------------------------------------------------
// One descriptor = one rectangle of a 2-D view: `rows` rows of `row_bytes` bytes, source rows `src_pitch` bytes apart,
// destination rows `dst_pitch` apart.  A tensor-parallel shard that becomes part of a differently sharded (or unsharded)
// tensor is one or a few such rectangles: a dim-0 shard is a block of whole rows, a dim-1 shard a column band of every
// row, a [q; k; v] or [gate; up] stacking three or two row blocks.  A work item is a group of rows of about 16 KB.
// QDQ: bf16 rows go through MXFP8 (1×32 blocks along the row, e8m0 scale) on the way, so the destination holds the values
// the block-quantised model would compute with; row_bytes must then be a multiple of 64.
struct Desc2 {
  long long src, dst, rows, row_bytes, src_pitch, dst_pitch;
};

__device__ __forceinline__ long long rows_per_item(long long row_bytes) {
  const long long r = kChunkBytes / (row_bytes > 0 ? row_bytes : 1);
  return r > 0 ? r : 1;
}

template <bool QDQ>
__global__ void __launch_bounds__(256) multi_copy2d_kernel(const Desc2* __restrict__ table, const long long* __restrict__ prefix, int n) {
  const long long total = prefix[n];
  for (long long c = blockIdx.x; c < total; c += gridDim.x) {
    const int d = find_desc(prefix, n, c);
    const Desc2 t = table[d];
    const long long rpi = rows_per_item(t.row_bytes);
    const long long r0 = (c - prefix[d]) * rpi;
    const long long r1 = min(t.rows, r0 + rpi);
    const bool vec = ((t.src | t.dst | t.row_bytes | t.src_pitch | t.dst_pitch) & 15) == 0;
    if (QDQ) {
      const long long blocks_per_row = t.row_bytes / 64;                 // 32 bf16 per block
      const long long items = (r1 - r0) * blocks_per_row;
      for (long long i = threadIdx.x; i < items; i += 256) {
        const long long r = r0 + i / blocks_per_row, b = i % blocks_per_row;
        const bf16* x = reinterpret_cast<const bf16*>(reinterpret_cast<const char*>(t.src) + r * t.src_pitch) + b * 32;
        bf16* y = reinterpret_cast<bf16*>(reinterpret_cast<char*>(t.dst) + r * t.dst_pitch) + b * 32;
        float v[32];
#pragma unroll
        for (int k = 0; k < 4; ++k) ld8(x + k * 8, v + k * 8);
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(v[k]));
        const int e = e8m0_for(amax);
        const float inv_scale = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);
        const float scale = __uint_as_float(static_cast<uint32_t>(max(e, 1)) << 23);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          __nv_bfloat162 o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_fp8x2_storage_t pair = __nv_cvt_float2_to_fp8x2(
                make_float2(v[8 * k + 2 * j] * inv_scale, v[8 * k + 2 * j + 1] * inv_scale), __NV_SATFINITE, __NV_E4M3);
            const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            o[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
          }
          reinterpret_cast<uint4*>(y)[k] = *reinterpret_cast<const uint4*>(o);
        }
      }
    } else if (vec) {
      const long long vpr = t.row_bytes >> 4;
      const long long items = (r1 - r0) * vpr;
      for (long long i = threadIdx.x; i < items; i += 256) {
        const long long r = r0 + i / vpr, v = i % vpr;
        reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.dst) + r * t.dst_pitch)[v] =
            reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(t.src) + r * t.src_pitch)[v];
      }
    } else {
      const long long items = (r1 - r0) * t.row_bytes;
      for (long long i = threadIdx.x; i < items; i += 256) {
        const long long r = r0 + i / t.row_bytes, b = i % t.row_bytes;
        (reinterpret_cast<char*>(t.dst) + r * t.dst_pitch)[b] = (reinterpret_cast<const char*>(t.src) + r * t.src_pitch)[b];
      }
    }
  }
}

int grid_for(long long total) { return static_cast<int>(total < 148 * 8 ? (total > 0 ? total : 1) : 148 * 8); }

}  // namespace
}  // namespace mb

// table: device int64 [n, 4] = {src, dst, bytes, 0}; prefix: device int64 [n+1] chunk offsets (16 KiB chunks); total = prefix[n]
extern "C" int mb_multi_copy(const long long* table, const long long* prefix, int n, long long total_chunks, cudaStream_t s) {
  if (n == 0 || total_chunks == 0) return 0;
  mb::multi_copy_kernel<<<mb::grid_for(total_chunks), 256, 0, s>>>(reinterpret_cast<const mb::Desc*>(table), prefix, n);
  return static_cast<int>(cudaGetLastError());
}

// table: {src bf16, dst (fp8 payload | bf16 when qdq), elements (multiple of 32), scale dst (unused when qdq)};
// prefix counts chunks of 256 blocks (8192 elements)
extern "C" int mb_multi_mxfp8(const long long* table, const long long* prefix, int n, long long total_chunks, int qdq,
                              cudaStream_t s) {
  if (n == 0 || total_chunks == 0) return 0;
  if (qdq)
    mb::multi_mxfp8_kernel<true><<<mb::grid_for(total_chunks), 256, 0, s>>>(reinterpret_cast<const mb::Desc*>(table), prefix, n);
  else
    mb::multi_mxfp8_kernel<false><<<mb::grid_for(total_chunks), 256, 0, s>>>(reinterpret_cast<const mb::Desc*>(table), prefix, n);
  return static_cast<int>(cudaGetLastError());
}

// table: device int64 [n, 6] = {src, dst, rows, row_bytes, src_pitch, dst_pitch}; prefix: device int64 [n+1] offsets of work items
// (a work item = max(1, 16384 / row_bytes) rows); qdq: rows go through MXFP8 on the way (bf16 in, bf16 out)
extern "C" int mb_multi_copy2d(const long long* table, const long long* prefix, int n, long long total_items, int qdq, cudaStream_t s) {
  if (n == 0 || total_items == 0) return 0;
  if (qdq)
    mb::multi_copy2d_kernel<true><<<mb::grid_for(total_items), 256, 0, s>>>(reinterpret_cast<const mb::Desc2*>(table), prefix, n);
  else
    mb::multi_copy2d_kernel<false><<<mb::grid_for(total_items), 256, 0, s>>>(reinterpret_cast<const mb::Desc2*>(table), prefix, n);
  return static_cast<int>(cudaGetLastError());
}
