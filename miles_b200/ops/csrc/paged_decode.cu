// Decode attention over a paged KV cache on tensor cores (flash-decoding with split keys).
//
// One CTA = (key split, KV head, request).  The `GROUP` query heads that share the KV head form the M dimension of
// mma.sync.m16n8k16 (rows ≥ GROUP are zero padding), so every K/V row fetched from HBM is used by all heads of the group
// and the score / PV products cost a handful of tensor-core instructions instead of per-key warp shuffles.
// K/V tiles of 64 keys are gathered from their cache pages with cp.async into XOR-swizzled shared memory, double
// buffered; each of the 4 warps owns 16 keys of a tile with its own running (max, sum, O) which are merged through
// shared memory at the end.  Split partials are combined by `paged_merge_kernel2`.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>

#include "launch.h"
#include "debug.cuh"
#include "pdl.cuh"

namespace mbpd {

typedef __nv_bfloat16 bf16;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr int TK = 64;  // keys per tile

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
template <int D>
__device__ __forceinline__ int toff(int row, int chunk) { return row * D + ((chunk ^ (row & 7)) << 3); }

template <int D>
__global__ void __launch_bounds__(128) paged_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                                                               const bf16* __restrict__ vc, const int* __restrict__ block_table,
                                                               const int* __restrict__ seq_lens, float* __restrict__ part_o,
                                                               float* __restrict__ part_ml, int max_blocks, int block_size, int Hq,
                                                               int Hkv, int group, float scale, int num_splits, bf16* __restrict__ out,
                                                               int* __restrict__ counters) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);   // 16 × D
  bf16* sK = sQ + 16 * D;                         // 2 × TK × D
  bf16* sV = sK + 2 * TK * D;                     // 2 × TK × D
  float* sM = reinterpret_cast<float*>(sV + 2 * TK * D);  // [4][8] max, [4][8] sum
  float* sL = sM + 32;
  float* sO = sL + 32;                            // [4][8][D]
  mb::pdl_trigger();
  mb::pdl_wait();
  const int req = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
  const int L = seq_lens[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kChunks = D / 8;
  const int per = ((L + num_splits - 1) / num_splits + TK - 1) / TK * TK;   // keys per split, whole tiles
  const int k_begin = split * per, k_end = min(L, k_begin + per);
  const int n_tiles = (k_end > k_begin) ? (k_end - k_begin + TK - 1) / TK : 0;
  const int* bt = block_table + static_cast<long long>(req) * max_blocks;

  // Q rows (heads of this group), zero padded to 16 rows
  for (int i = threadIdx.x; i < 16 * kChunks; i += 128) {
    const int r = i / kChunks, c = i % kChunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < group) v = *reinterpret_cast<const uint4*>(q + (static_cast<long long>(req) * Hq + hk * group + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + toff<D>(r, c)) = v;
  }
  auto load_tile = [&](int t, int st) {
    const int k0 = k_begin + t * TK;
    for (int i = threadIdx.x; i < TK * kChunks; i += 128) {
      const int r = i / kChunks, c = i % kChunks;
      const int key = k0 + r;
      bool ok = key < k_end;
      const int kk = ok ? key : k_begin;
      long long blk = bt[kk / block_size];
      if (!mb::dbg::in_bounds(mb::dbg::kKvBlocks, blk, 301)) { ok = false; blk = 0; }   // debug build: zero-filled instead of read
      const long long slot = blk * block_size + kk % block_size;
      const long long off = (slot * Hkv + hk) * D + c * 8;
      cp_async16(sK + st * TK * D + toff<D>(r, c), kc + off, ok);
      cp_async16(sV + st * TK * D + toff<D>(r, c), vc + off, ok);
    }
    cp_async_commit();
  };
  if (n_tiles > 0) load_tile(0, 0);
  __syncthreads();
  // Q fragments stay in registers
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int row = lane & 15, chunk = ks * 2 + (lane >> 4);
    ldsm_x4(s_addr(sQ + toff<D>(row, chunk)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_i = -INFINITY, l_i = 0.f;   // row lane/4 (the rows lane/4 + 8 are padding)
  const float sl2 = scale * kLog2e;

  for (int t = 0; t < n_tiles; ++t) {
    const int st = t & 1;
    if (t + 1 < n_tiles) {
      load_tile(t + 1, st ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + st * TK * D;
    const bf16* tV = sV + st * TK * D;
    const int key0 = k_begin + t * TK + warp * 16;
    if (key0 < k_end) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b[4];
        const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        ldsm_x4(s_addr(tK + toff<D>(row, chunk)), b[0], b[1], b[2], b[3]);
        mma16816(s[0], qa[ks], b[0], b[1]);
        mma16816(s[1], qa[ks], b[2], b[3]);
      }
      float mx = m_i;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + nt * 8 + (lane & 3) * 2 + e;
          if (key >= k_end) s[nt][e] = -INFINITY;
          mx = fmaxf(mx, s[nt][e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float msc = (mx == -INFINITY) ? 0.f : mx * sl2;
      const float alpha = (m_i == -INFINITY) ? 0.f : exp2f(m_i * sl2 - msc);
      m_i = mx;
      float rs = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float p = exp2f(s[nt][e] * sl2 - msc);
          s[nt][e] = p;
          rs += p;
        }
      l_i = l_i * alpha + rs;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o_acc[i][0] *= alpha; o_acc[i][1] *= alpha; }
      // P (rows 0..7 real, rows 8..15 zero) as the A operand for 16 keys
      const uint32_t pa[4] = {pack2(s[0][0], s[0][1]), 0u, pack2(s[1][0], s[1][1]), 0u};
#pragma unroll
      for (int nc = 0; nc < D / 16; ++nc) {
        uint32_t b[4];
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int chunk = nc * 2 + (lane >> 4);
        ldsm_x4_t(s_addr(tV + toff<D>(row, chunk)), b[0], b[1], b[2], b[3]);
        mma16816(o_acc[2 * nc], pa, b[0], b[1]);
        mma16816(o_acc[2 * nc + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  // merge the four warps (each holds rows 0..7 in lanes' c0/c1)
  l_i += __shfl_xor_sync(0xffffffffu, l_i, 1);
  l_i += __shfl_xor_sync(0xffffffffu, l_i, 2);
  const int r = lane >> 2;
  if ((lane & 3) == 0) { sM[warp * 8 + r] = m_i; sL[warp * 8 + r] = l_i; }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    sO[(warp * 8 + r) * D + i * 8 + (lane & 3) * 2] = o_acc[i][0];
    sO[(warp * 8 + r) * D + i * 8 + (lane & 3) * 2 + 1] = o_acc[i][1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < group * D; i += 128) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sM[w * 8 + g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sM[w * 8 + g];
      const float a = (mw == -INFINITY) ? 0.f : exp2f((mw - mm) * sl2);
      ll += sL[w * 8 + g] * a;
      oo += sO[(w * 8 + g) * D + d] * a;
    }
    const long long base = (static_cast<long long>(req) * Hq + hk * group + g) * num_splits + split;
    if (counters != nullptr && num_splits == 1) {          // a single split: normalise and write the result directly
      out[(static_cast<long long>(req) * Hq + hk * group + g) * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
      continue;
    }
    __stcg(&part_o[base * D + d], oo);
    if (d == 0) { __stcg(&part_ml[base * 2], (mm == -INFINITY) ? -INFINITY : mm * sl2); __stcg(&part_ml[base * 2 + 1], ll); }
  }
  if (counters == nullptr || num_splits == 1) return;      // merged by paged_merge_kernel2 / nothing to merge
  // the last split of this (request, kv head) to arrive merges all of them: no second kernel
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[req * Hkv + hk], 1) == num_splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < group * D; i += 128) {
    const int g = i / D, d = i % D;
    const long long rh = static_cast<long long>(req) * Hq + hk * group + g;
    float mm = -INFINITY;
    for (int sp = 0; sp < num_splits; ++sp) mm = fmaxf(mm, __ldcg(&part_ml[(rh * num_splits + sp) * 2]));
    float ll = 0.f, oo = 0.f;
    for (int sp = 0; sp < num_splits; ++sp) {
      const float ms = __ldcg(&part_ml[(rh * num_splits + sp) * 2]);
      const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      ll += __ldcg(&part_ml[(rh * num_splits + sp) * 2 + 1]) * a;
      oo += __ldcg(&part_o[(rh * num_splits + sp) * D + d]) * a;
    }
    out[rh * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
  }
  if (threadIdx.x == 0) counters[req * Hkv + hk] = 0;
}

// partial maxima are stored pre-multiplied by scale·log2(e)
template <int D>
__global__ void paged_merge_kernel2(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    int num_splits) {
  mb::pdl_trigger();
  mb::pdl_wait();
  const long long rh = blockIdx.x;
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
static size_t smem_bytes() { return static_cast<size_t>(16 * D + 4 * TK * D) * 2 + 64 * sizeof(float) + 4 * 8 * D * sizeof(float); }

}  // namespace mbpd

using namespace mbpd;

MB_DEFINE_BOUNDS_API(mb_paged_bounds)

// part_o: [B·Hq·splits·D] floats, part_ml: [B·Hq·splits·2] floats.  Hq/Hkv ≤ 8.
extern "C" int mb_paged_decode(const void* q, const void* kc, const void* vc, const int* block_table, const int* seq_lens, void* out,
                               float* part_o, float* part_ml, int batch, int max_blocks, int block_size, int Hq, int Hkv, int D,
                               float scale, int num_splits, cudaStream_t s) {
  if (batch == 0) return 0;
  const int group = Hq / Hkv;
  if (group > 8 || group * Hkv != Hq) return -2;
  dim3 grid(num_splits, Hkv, batch);
  // Optional in-kernel merge (MILES_DECODE_FUSED_MERGE=1): the last split of a (request, kv head) to arrive merges them,
  // which saves the merge launch but leaves the whole GQA group to one CTA; measured slower than the separate merge
  // kernel at the batch sizes of the rollout (21 µs against 11 + 4 µs at batch 8), so it is off by default.
  // Arrival counters: one per (request, kv head), zero between calls; allocated on first use outside stream capture.
  static const bool fused_merge = [] { const char* e = getenv("MILES_DECODE_FUSED_MERGE"); return e != nullptr && e[0] == '1'; }();
  static int* counter_buf[64] = {};
  static int counter_cap[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int* counters = nullptr;
  if (fused_merge && dev < 64) {
    if (counter_cap[dev] < batch * Hkv) {
      cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing(s, &st);
      if (st == cudaStreamCaptureStatusNone) {
        const int cap = batch * Hkv > 16384 ? batch * Hkv : 16384;
        int* fresh = nullptr;
        if (cudaMalloc(&fresh, cap * sizeof(int)) == cudaSuccess && cudaMemset(fresh, 0, cap * sizeof(int)) == cudaSuccess) {
          counter_buf[dev] = fresh;      // an older, smaller buffer may still be referenced by captured graphs: it is kept
          counter_cap[dev] = cap;
        }
      }
    }
    if (counter_cap[dev] >= batch * Hkv) counters = counter_buf[dev];
  }
  bf16* O = reinterpret_cast<bf16*>(out);
  auto Q = reinterpret_cast<const bf16*>(q);
  auto KC = reinterpret_cast<const bf16*>(kc);
  auto VC = reinterpret_cast<const bf16*>(vc);
  if (D == 128) {
    static bool once = false;
    if (!once) {
      cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_bytes<128>()));
      if (e != cudaSuccess) return static_cast<int>(e);
      once = true;
    }
    cudaError_t e = mb::launch_pdl(paged_decode_mma_kernel<128>, grid, dim3(128), smem_bytes<128>(), s, Q, KC, VC, block_table, seq_lens, part_o,
                               part_ml, max_blocks, block_size, Hq, Hkv, group, scale, num_splits, O, counters);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (counters == nullptr) e = mb::launch_pdl(paged_merge_kernel2<128>, dim3(batch * Hq), dim3(128), 0, s, static_cast<const float*>(part_o),
                   static_cast<const float*>(part_ml), reinterpret_cast<bf16*>(out), num_splits);
    if (e != cudaSuccess) return static_cast<int>(e);
  } else if (D == 64) {
    static bool once = false;
    if (!once) {
      cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem_bytes<64>()));
      if (e != cudaSuccess) return static_cast<int>(e);
      once = true;
    }
    cudaError_t e = mb::launch_pdl(paged_decode_mma_kernel<64>, grid, dim3(128), smem_bytes<64>(), s, Q, KC, VC, block_table, seq_lens, part_o,
                               part_ml, max_blocks, block_size, Hq, Hkv, group, scale, num_splits, O, counters);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (counters == nullptr) e = mb::launch_pdl(paged_merge_kernel2<64>, dim3(batch * Hq), dim3(64), 0, s, static_cast<const float*>(part_o),
                   static_cast<const float*>(part_ml), reinterpret_cast<bf16*>(out), num_splits);
    if (e != cudaSuccess) return static_cast<int>(e);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}
