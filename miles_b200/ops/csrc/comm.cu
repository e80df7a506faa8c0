// Compute kernels that read or write peer GPUs' memory directly (NVLink peer pointers), plus the cross-rank barrier.
//   barrier                 flag exchange between all ranks (release/acquire at system scope, bounded waits)
//   ar_add_rmsnorm          one-shot all-reduce of per-rank partial rows fused with residual add + RMSNorm
//   rs_reduce_sqnorm        this rank's shard = Σ over ranks of their fp32 gradient buffers (peer loads) + Σ g²
//   adam_allgather          AdamW on the shard, new bf16 parameters stored into every rank's parameter buffer
//   moe_dispatch            token rows pushed into the owning rank's receive buffer (remote atomic row allocation)
//   moe_scatter_known       rows pushed to remote rows that are already known (backward of dispatch)
//   moe_return              expert outputs pushed back into the source rank's per-(token, slot) return buffer
//   stats_merge             vocab-parallel log-prob: merge every rank's (max, Σexp, Σexp·z, target) rows
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "launch.h"
#include "pdl.cuh"

namespace mb {

typedef __nv_bfloat16 bf16;

// The epoch comes from a device-side counter that every rank advances identically (same launch sequence), so the
// kernel can be replayed from a CUDA graph without a host-provided epoch.
__global__ void barrier_kernel(PeerPtrs flags, int rank, int world, int channel, int* epochs, int* err) {
  __shared__ int epoch_sh;
  if (threadIdx.x == 0) epoch_sh = ++epochs[channel];
  __syncthreads();
  if (!cross_rank_barrier(flags, rank, world, channel, epoch_sh)) {
    if (threadIdx.x == 0) atomicExch(err, 100 + channel);
  }
}

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_256(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) r += sh[i];
  return r;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(h[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return o;
}

// y = rmsnorm(Σ_r partial_r + residual)·w ; res_out = Σ_r partial_r + residual.  One CTA per row, H ≤ 8192, H % 8 == 0.
__global__ void __launch_bounds__(256) ar_add_rmsnorm_kernel(PeerPtrs partials, int world, const bf16* __restrict__ residual,
                                                             const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ res_out,
                                                             int H, float eps) {
  if (fabric_poisoned()) return;
  __shared__ float sh[8];
  const long long row = blockIdx.x;
  const int nvec = H / 8;
  float acc[4][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int v = threadIdx.x + it * 256;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[it][i] = 0.f;
      for (int r = 0; r < world; ++r) {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(partials.p[r]) + row * H + v * 8);
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[it][i] += f[i];
      }
      if (residual != nullptr) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(residual + row * H + v * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[it][i] += f[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[it][i] = __bfloat162float(__float2bfloat16(acc[it][i]));
      if (res_out != nullptr) *reinterpret_cast<uint4*>(res_out + row * H + v * 8) = pack8(acc[it]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += acc[it][i] * acc[it][i];
    }
  }
  ss = block_sum_256(ss, sh);
  const float rstd = rsqrtf(ss / H + eps);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int v = threadIdx.x + it * 256;
    if (v < nvec) {
      float wv[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(w + v * 8), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = acc[it][i] * rstd * wv[i];
      *reinterpret_cast<uint4*>(y + row * H + v * 8) = pack8(o);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out[i] (local, i in [lo, hi)) = Σ_r grads_r[i]; sqnorm += Σ out[i]²·weight[i]  (weight: 0 for entries another
// rank also counts, e.g. tensor-parallel replicas; nullptr → 1)
__global__ void __launch_bounds__(256) rs_reduce_sqnorm_kernel(PeerPtrs grads, int world, int rank, long long lo, long long hi,
                                                               const float* __restrict__ norm_weight, float* __restrict__ sqnorm) {
  if (fabric_poisoned()) return;
  __shared__ float sh[8];
  float ss = 0.f;
  float* mine = reinterpret_cast<float*>(grads.p[rank]);
  for (long long i = lo + (blockIdx.x * 256ll + threadIdx.x) * 4; i < hi; i += static_cast<long long>(gridDim.x) * 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + i);
      acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
    }
    *reinterpret_cast<float4*>(mine + i) = acc;
    float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
    if (norm_weight != nullptr) nw = *reinterpret_cast<const float4*>(norm_weight + (i - lo));
    ss += acc.x * acc.x * nw.x + acc.y * acc.y * nw.y + acc.z * acc.z * nw.z + acc.w * acc.w * nw.w;
  }
  ss = block_sum_256(ss, sh);
  if (threadIdx.x == 0) atomicAdd(sqnorm, ss);
}

// AdamW on the local shard [lo, hi) of the (already reduced) gradient; the updated bf16 parameters are stored into
// every rank's parameter buffer at the same offsets (the all-gather).  clip: scale = min(1, clip / (sqrt(*sqnorm) + 1e-6)).
__global__ void __launch_bounds__(256) adam_allgather_kernel(float* __restrict__ master, const float* __restrict__ grad_shard,
                                                             float* __restrict__ m, float* __restrict__ v,
                                                             const float* __restrict__ decay_mask, const float* __restrict__ sqnorm,
                                                             float clip, PeerPtrs params, int world, long long lo, long long n, float lr,
                                                             float b1, float b2, float eps, float wd, float bc1, float bc2) {
  if (fabric_poisoned()) return;
  float scale = 1.f;
  if (clip > 0.f && sqnorm != nullptr) scale = fminf(1.f, clip / (sqrtf(*sqnorm) + 1e-6f));
  for (long long i = (blockIdx.x * 256ll + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * 1024) {
    float4 g = *reinterpret_cast<const float4*>(grad_shard + i);
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
      pp[k] = pp[k] * (1.f - lr * wd * dp[k]) - lr * (mp[k] / bc1) / (sqrtf(vp[k] / bc2) + eps);
    }
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    *reinterpret_cast<float4*>(master + i) = p;
    uint2 o;
    __nv_bfloat162 lo2 = __floats2bfloat162_rn(pp[0], pp[1]);
    __nv_bfloat162 hi2 = __floats2bfloat162_rn(pp[2], pp[3]);
    o.x = *reinterpret_cast<uint32_t*>(&lo2);
    o.y = *reinterpret_cast<uint32_t*>(&hi2);
    for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(params.p[r]) + lo + i) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// MoE dispatch.  One warp per (token, slot) pair: the destination rank is expert / e_local; lane 0 allocates a row in the
// destination's receive buffer with a remote atomicAdd on that rank's counter, then the warp copies the token row and
// writes the metadata {source rank, source flat index, local expert id}.  sent_dest/sent_row remember the placement.
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ topk_idx, long long n_pairs,
                                                           int k, int H, int e_local, int rank, PeerPtrs recv_x, PeerPtrs recv_meta,
                                                           PeerPtrs counters, int capacity, int* __restrict__ sent_row, int* err,
                                                           int world) {
  if (fabric_poisoned()) return;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  for (long long pair = (blockIdx.x * 256ll + threadIdx.x) >> 5; pair < n_pairs; pair += (static_cast<long long>(gridDim.x) * 256) >> 5) {
    const int e = topk_idx[pair];
    if (e < 0) {
      if (lane == 0) sent_row[pair] = -1;
      continue;
    }
    if (e >= e_local * world) {
      // an expert id no rank owns (a router row of NaNs, a corrupt replay record): the peer table must not be indexed with it
      if (lane == 0) { atomicCAS(err, 0, 210); sent_row[pair] = -1; }
      continue;
    }
    const int dest = e / e_local;
    int row = 0;
    if (lane == 0) row = atomicAdd(reinterpret_cast<int*>(counters.p[dest]), 1);
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row >= capacity) {
      if (lane == 0) { atomicExch(err, 200); sent_row[pair] = -1; }
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (pair / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv_x.p[dest]) + static_cast<long long>(row) * H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
    if (lane == 0) {
      int4 meta = make_int4(rank, static_cast<int>(pair), e - dest * e_local, 0);
      reinterpret_cast<int4*>(recv_meta.p[dest])[row] = meta;
      sent_row[pair] = row;
    }
  }
}

// Decode-time expert parallelism with the barriers folded into the kernels on either side of them (inference, at most
// 16384 receivable rows): `moe_dispatch_signal` = dispatch + publish from its last block; `moe_recv_align` = wait for every
// peer's publish, read and reset the receive counter, counting-sort the received rows by local expert;
// `moe_return_signal` = return + publish; `moe_combine_wait` = wait + weighted sum.  Four launches where the general path
// takes eight (dispatch, barrier, expert-id scan, align, …, return, barrier, combine).
__global__ void __launch_bounds__(256) moe_dispatch_signal_kernel(const bf16* __restrict__ x, const int* __restrict__ topk_idx,
                                                                  long long n_pairs, int k, int H, int e_local, int rank,
                                                                  PeerPtrs recv_x, PeerPtrs recv_meta, PeerPtrs counters, int capacity,
                                                                  int* __restrict__ sent_row, int* err, PeerPtrs flags, int world,
                                                                  int channel, int* epochs, int* ticket) {
  // programmatic dependent launch: the successor may be scheduled at once (it waits for this grid's completion before it
  // reads anything), and nothing a predecessor wrote is read here before the wait
  pdl_trigger();
  pdl_wait();
  if (!fabric_poisoned()) {
    const int lane = threadIdx.x & 31;
    const int nvec = H / 8;
    for (long long pair = (blockIdx.x * 256ll + threadIdx.x) >> 5; pair < n_pairs; pair += (static_cast<long long>(gridDim.x) * 256) >> 5) {
      const int e = topk_idx[pair];
      if (e < 0) {
        if (lane == 0) sent_row[pair] = -1;
        continue;
      }
      if (e >= e_local * world) {
        if (lane == 0) { atomicCAS(err, 0, 210); sent_row[pair] = -1; }
        continue;
      }
      const int dest = e / e_local;
      int row = 0;
      if (lane == 0) row = atomicAdd(reinterpret_cast<int*>(counters.p[dest]), 1);
      row = __shfl_sync(0xffffffffu, row, 0);
      if (row >= capacity) {
        if (lane == 0) { atomicCAS(err, 0, 200); sent_row[pair] = -1; }
        continue;
      }
      const uint4* src = reinterpret_cast<const uint4*>(x + (pair / k) * H);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv_x.p[dest]) + static_cast<long long>(row) * H);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      if (lane == 0) {
        reinterpret_cast<int4*>(recv_meta.p[dest])[row] = make_int4(rank, static_cast<int>(pair), e - dest * e_local, 0);
        sent_row[pair] = row;
      }
    }
  }
  publish_when_grid_done(flags, rank, world, channel, epochs, ticket);
}

// One block.  Outputs as `moe_align`: seg_offsets[E+1] (segments padded to `pad`), tile_expert[max_rows / pad], row_src[max_rows].
__global__ void __launch_bounds__(1024) moe_recv_align_kernel(const int4* __restrict__ meta, int* __restrict__ counter, int capacity, int E,
                                                              int* __restrict__ seg_offsets, int* __restrict__ tile_expert,
                                                              int* __restrict__ row_src, int max_rows, int pad, PeerPtrs flags, int rank,
                                                              int world, int channel, const int* epochs, int* err) {
  extern __shared__ int sh[];   // counts[E], cursor[E], seg[E+1], n
  int* counts = sh;
  int* cursor = sh + E;
  int* seg = sh + 2 * E;
  int* n_sh = sh + 3 * E + 1;
  pdl_trigger();
  pdl_wait();
  const bool ok = wait_peers(flags, rank, world, channel, epochs);
  if (!ok && threadIdx.x == 0) atomicCAS(err, 0, 100 + channel);
  if (threadIdx.x == 0) *n_sh = ok ? min(*counter, capacity) : 0;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  __syncthreads();
  const int n = *n_sh;
  if (threadIdx.x == 0) *counter = 0;      // peers add to it again only after the next publish of this rank's stream
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = meta[i].z;
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
      int lo = 0, hi = E;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
    }
    tile_expert[t] = ex;
  }
  for (int r = threadIdx.x; r < seg[E] && r < max_rows; r += blockDim.x) row_src[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = meta[i].z;
    if (e >= 0 && e < E) {
      const int row = seg[e] + atomicAdd(&cursor[e], 1);
      if (row < max_rows) row_src[row] = i;
    }
  }
}

__global__ void __launch_bounds__(256) moe_return_signal_kernel(const bf16* __restrict__ y_perm, const int* __restrict__ row_src,
                                                                const int4* __restrict__ meta, const int* __restrict__ seg_offsets, int E,
                                                                int H, int max_rows, PeerPtrs ret, PeerPtrs flags, int rank, int world,
                                                                int channel, int* epochs, int* ticket) {
  pdl_trigger();
  pdl_wait();
  if (!fabric_poisoned()) {
    const int lane = threadIdx.x & 31;
    const int nvec = H / 8;
    const int total = min(seg_offsets[E], max_rows);
    for (int p = (blockIdx.x * 256 + threadIdx.x) >> 5; p < total; p += (gridDim.x * 256) >> 5) {
      const int r = row_src[p];
      if (r < 0) continue;
      const int4 mt = meta[r];
      const uint4* src = reinterpret_cast<const uint4*>(y_perm + static_cast<long long>(p) * H);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(ret.p[mt.x]) + static_cast<long long>(mt.y) * H);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
    }
  }
  publish_when_grid_done(flags, rank, world, channel, epochs, ticket);
}

// out[t, :] = Σ_j w[t, j] · ret[t·k + j, :] over the pairs that took part (sent_row ≥ 0), after every peer's publish arrived
__global__ void __launch_bounds__(256) moe_combine_wait_kernel(const bf16* __restrict__ ret, const float* __restrict__ w,
                                                               const int* __restrict__ sent_row, bf16* __restrict__ out, long long T, int k,
                                                               int H, PeerPtrs flags, int rank, int world, int channel, const int* epochs,
                                                               int* err) {
  // the next kernel of the stream (the following layer's fused norm + projection) is released at once: it streams its
  // weights while this grid still waits for the peers' results
  pdl_trigger();
  pdl_wait();
  if (!wait_peers(flags, rank, world, channel, epochs)) {
    if (threadIdx.x == 0) atomicCAS(err, 0, 100 + channel);
    return;
  }
  if (fabric_poisoned()) return;
  const int nvec = H / 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    for (int v = threadIdx.x; v < nvec; v += 256) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; ++j) {
        if (sent_row[t * k + j] < 0) continue;
        const float wj = w[t * k + j];
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(ret + (t * k + j) * H + v * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += wj * f[i];
      }
      *reinterpret_cast<uint4*>(out + t * H + v * 8) = pack8(acc);
    }
  }
}

// Rows pushed to remote rows that are already known: dst rank = topk_idx / e_local, dst row = sent_row[pair].
// rows_in is indexed by pair (src_by_pair = 1) or by token (pair / k).
__global__ void __launch_bounds__(256) moe_scatter_known_kernel(const bf16* __restrict__ rows_in, int src_by_pair,
                                                                const int* __restrict__ topk_idx, const int* __restrict__ sent_row,
                                                                long long n_pairs, int k, int H, int e_local, PeerPtrs recv_x) {
  if (fabric_poisoned()) return;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  for (long long pair = (blockIdx.x * 256ll + threadIdx.x) >> 5; pair < n_pairs; pair += (static_cast<long long>(gridDim.x) * 256) >> 5) {
    const int row = sent_row[pair];
    if (row < 0) continue;
    const int dest = topk_idx[pair] / e_local;
    const uint4* src = reinterpret_cast<const uint4*>(rows_in + (src_by_pair ? pair : pair / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv_x.p[dest]) + static_cast<long long>(row) * H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
}

// Expert outputs back to their source: for permuted row p with receive-row r = row_src[p] ≥ 0 and meta[r] = {src rank,
// src pair, …}: ret_{src rank}[src pair, :] = y_perm[p, :].
__global__ void __launch_bounds__(256) moe_return_kernel(const bf16* __restrict__ y_perm, const int* __restrict__ row_src,
                                                         const int4* __restrict__ meta, const int* __restrict__ seg_offsets, int E,
                                                         int H, int max_rows, PeerPtrs ret) {
  if (fabric_poisoned()) return;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  const int total = min(seg_offsets[E], max_rows);
  for (int p = (blockIdx.x * 256 + threadIdx.x) >> 5; p < total; p += (gridDim.x * 256) >> 5) {
    const int r = row_src[p];
    if (r < 0) continue;
    const int4 mt = meta[r];
    const uint4* src = reinterpret_cast<const uint4*>(y_perm + static_cast<long long>(p) * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(ret.p[mt.x]) + static_cast<long long>(mt.y) * H);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
}

// Local expert id per received row (for the counting sort), from the metadata; n is read from the device counter.
// clear_counter (single-block launches only): the receive counter is reset here, after every thread has its copy of n,
// instead of by a separate memset; peers only add to it again after the next cross-rank barrier of the stream.
__global__ void recv_expert_ids_kernel(const int4* __restrict__ meta, int* __restrict__ counter, int capacity,
                                       int* __restrict__ expert_ids, int* __restrict__ n_out, int clear_counter) {
  __shared__ int n_sh;
  if (threadIdx.x == 0) n_sh = min(*counter, capacity);
  __syncthreads();
  const int n = n_sh;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *n_out = n;
    if (clear_counter) *counter = 0;
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x)
    expert_ids[i] = (i < n) ? meta[i].z : -1;
}

// ---------------------------------------------------------------------------------------------
// Vocab-parallel log-prob: merge the per-rank streaming statistics {m, s, e, t} (see misc.cu) of every rank.
// A rank whose vocabulary shard does not contain the target leaves t = 0 and contributes nothing to it.
__global__ void stats_merge_kernel(PeerPtrs stats, int world, long long R, float* __restrict__ logp, float* __restrict__ ent,
                                   float* __restrict__ lse) {
  if (fabric_poisoned()) return;
  const long long r = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (r >= R) return;
  float M = -INFINITY, S = 0.f, Es = 0.f, T = 0.f;
  for (int k = 0; k < world; ++k) {
    const float4 st = reinterpret_cast<const float4*>(stats.p[k])[r];
    const float nm = fmaxf(M, st.x);
    const float a = (M == -INFINITY) ? 0.f : __expf(M - nm), b = (st.x == -INFINITY) ? 0.f : __expf(st.x - nm);
    S = S * a + st.y * b;
    Es = Es * a + st.z * b;
    M = nm;
    T += st.w;
  }
  const float l = M + __logf(S);
  logp[r] = T - l;
  if (ent != nullptr) ent[r] = l - Es / S;
  if (lse != nullptr) lse[r] = l;
}

// out[i] = Σ_r src_r[i] (bf16, fp32 accumulate): every rank reads the same-shaped block from each peer.
__global__ void __launch_bounds__(256) sum_rows_kernel(PeerPtrs src, int world, bf16* __restrict__ out, long long nvec) {
  if (fabric_poisoned()) return;
  for (long long v = blockIdx.x * 256ll + threadIdx.x; v < nvec; v += static_cast<long long>(gridDim.x) * 256) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(src.p[r])[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    reinterpret_cast<uint4*>(out)[v] = pack8(acc);
  }
}

// out[r·n + i] = src_r[i]: all-gather by peer loads (16-byte vectors), n = elements per rank / 8.
__global__ void __launch_bounds__(256) gather_rows_kernel(PeerPtrs src, int world, uint4* __restrict__ out, long long nvec_per_rank) {
  if (fabric_poisoned()) return;
  const long long total = nvec_per_rank * world;
  for (long long v = blockIdx.x * 256ll + threadIdx.x; v < total; v += static_cast<long long>(gridDim.x) * 256) {
    const int r = static_cast<int>(v / nvec_per_rank);
    out[v] = reinterpret_cast<const uint4*>(src.p[r])[v - r * nvec_per_rank];
  }
}

static PeerPtrs make_ptrs(const long long* ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = (i < world) ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

static int blocks_for(long long items, int per_block, int cap = 148 * 4) {
  long long b = (items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<int>(b);
}

}  // namespace mb

using namespace mb;

MB_DEFINE_FABRIC_CONFIGURE(mb_comm_configure)

extern "C" int mb_barrier(const long long* flag_ptrs, int rank, int world, int channel, int* epochs, int* err, cudaStream_t s) {
  if (world > kMaxRanks) return -1;
  barrier_kernel<<<1, 32, 0, s>>>(make_ptrs(flag_ptrs, world), rank, world, channel, epochs, err);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_ar_add_rmsnorm(const long long* partial_ptrs, int world, const void* residual, const void* w, void* y,
                                 void* res_out, long long T, int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 || H > 8192 || world > kMaxRanks) return -1;
  ar_add_rmsnorm_kernel<<<static_cast<unsigned>(T), 256, 0, s>>>(make_ptrs(partial_ptrs, world), world,
                                                                 reinterpret_cast<const bf16*>(residual), reinterpret_cast<const bf16*>(w),
                                                                 reinterpret_cast<bf16*>(y), reinterpret_cast<bf16*>(res_out), H, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_rs_reduce_sqnorm(const long long* grad_ptrs, int world, int rank, long long lo, long long hi,
                                   const float* norm_weight, float* sqnorm, cudaStream_t s) {
  if (hi <= lo) return 0;
  if ((lo % 4) || (hi % 4)) return -1;
  rs_reduce_sqnorm_kernel<<<blocks_for(hi - lo, 1024, 148 * 8), 256, 0, s>>>(make_ptrs(grad_ptrs, world), world, rank, lo, hi,
                                                                           norm_weight, sqnorm);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_adam_allgather(float* master, const float* grad_shard, float* m, float* v, const float* decay_mask,
                                 const float* sqnorm, float clip, const long long* param_ptrs, int world, long long lo, long long n,
                                 float lr, float b1, float b2, float eps, float wd, int step, cudaStream_t s) {
  if (n == 0) return 0;
  if ((lo % 4) || (n % 4)) return -1;
  const float bc1 = 1.f - powf(b1, static_cast<float>(step)), bc2 = 1.f - powf(b2, static_cast<float>(step));
  adam_allgather_kernel<<<blocks_for(n, 1024, 148 * 8), 256, 0, s>>>(master, grad_shard, m, v, decay_mask, sqnorm, clip,
                                                                   make_ptrs(param_ptrs, world), world, lo, n, lr, b1, b2, eps, wd,
                                                                   bc1, bc2);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_moe_dispatch(const void* x, const int* topk_idx, long long n_pairs, int k, int H, int e_local, int rank,
                               const long long* recv_x_ptrs, const long long* recv_meta_ptrs, const long long* counter_ptrs, int world,
                               int capacity, int* sent_row, int* err, cudaStream_t s) {
  if (n_pairs == 0) return 0;
  if (H % 8) return -1;
  moe_dispatch_kernel<<<blocks_for(n_pairs, 8), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), topk_idx, n_pairs, k, H, e_local, rank,
                                                             make_ptrs(recv_x_ptrs, world), make_ptrs(recv_meta_ptrs, world),
                                                             make_ptrs(counter_ptrs, world), capacity, sent_row, err, world);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_moe_dispatch_signal(const void* x, const int* topk_idx, long long n_pairs, int k, int H, int e_local, int rank,
                                      const long long* recv_x_ptrs, const long long* recv_meta_ptrs, const long long* counter_ptrs,
                                      int world, int capacity, int* sent_row, int* err, const long long* flag_ptrs, int channel,
                                      int* epochs, int* ticket, cudaStream_t s) {
  if (H % 8 || world > kMaxRanks) return -1;
  return static_cast<int>(launch_pdl(moe_dispatch_signal_kernel, dim3(blocks_for(n_pairs > 0 ? n_pairs : 1, 8)), dim3(256), 0, s,
                                     reinterpret_cast<const bf16*>(x), topk_idx, n_pairs, k, H, e_local, rank,
                                     make_ptrs(recv_x_ptrs, world), make_ptrs(recv_meta_ptrs, world), make_ptrs(counter_ptrs, world),
                                     capacity, sent_row, err, make_ptrs(flag_ptrs, world), world, channel, epochs, ticket));
}

extern "C" int mb_moe_recv_align(const void* meta, int* counter, int capacity, int E, int* seg_offsets, int* tile_expert, int* row_src,
                                 int max_rows, int pad, const long long* flag_ptrs, int rank, int world, int channel, const int* epochs,
                                 int* err, cudaStream_t s) {
  if (capacity > 16384 || world > kMaxRanks || pad <= 0 || max_rows % pad) return -1;
  return static_cast<int>(launch_pdl(moe_recv_align_kernel, dim3(1), dim3(1024), (3 * E + 2) * sizeof(int), s,
                                     reinterpret_cast<const int4*>(meta), counter, capacity, E, seg_offsets, tile_expert, row_src,
                                     max_rows, pad, make_ptrs(flag_ptrs, world), rank, world, channel, epochs, err));
}

extern "C" int mb_moe_return_signal(const void* y_perm, const int* row_src, const void* meta, const int* seg_offsets, int E, int H,
                                    int max_rows, const long long* ret_ptrs, int world, const long long* flag_ptrs, int rank, int channel,
                                    int* epochs, int* ticket, cudaStream_t s) {
  if (world > kMaxRanks) return -1;
  return static_cast<int>(launch_pdl(moe_return_signal_kernel, dim3(blocks_for(max_rows > 0 ? max_rows : 1, 8)), dim3(256), 0, s,
                                     reinterpret_cast<const bf16*>(y_perm), row_src, reinterpret_cast<const int4*>(meta), seg_offsets,
                                     E, H, max_rows, make_ptrs(ret_ptrs, world), make_ptrs(flag_ptrs, world), rank, world, channel,
                                     epochs, ticket));
}

extern "C" int mb_moe_combine_wait(const void* ret, const float* w, const int* sent_row, void* out, long long T, int k, int H,
                                   const long long* flag_ptrs, int rank, int world, int channel, const int* epochs, int* err,
                                   cudaStream_t s) {
  if (H % 8 || world > kMaxRanks) return -1;
  const int blocks = T < 1 ? 1 : (T < 148 * 16 ? static_cast<int>(T) : 148 * 16);
  return static_cast<int>(launch_pdl(moe_combine_wait_kernel, dim3(blocks), dim3(256), 0, s, reinterpret_cast<const bf16*>(ret), w,
                                     sent_row, reinterpret_cast<bf16*>(out), T, k, H, make_ptrs(flag_ptrs, world), rank, world,
                                     channel, epochs, err));
}

extern "C" int mb_moe_scatter_known(const void* rows_in, int src_by_pair, const int* topk_idx, const int* sent_row, long long n_pairs,
                                    int k, int H, int e_local, const long long* recv_x_ptrs, int world, cudaStream_t s) {
  if (n_pairs == 0) return 0;
  moe_scatter_known_kernel<<<blocks_for(n_pairs, 8), 256, 0, s>>>(reinterpret_cast<const bf16*>(rows_in), src_by_pair, topk_idx, sent_row,
                                                                  n_pairs, k, H, e_local, make_ptrs(recv_x_ptrs, world));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_moe_return(const void* y_perm, const int* row_src, const void* meta, const int* seg_offsets, int E, int H,
                             int max_rows, const long long* ret_ptrs, int world, cudaStream_t s) {
  if (max_rows == 0) return 0;
  moe_return_kernel<<<blocks_for(max_rows, 8), 256, 0, s>>>(reinterpret_cast<const bf16*>(y_perm), row_src,
                                                            reinterpret_cast<const int4*>(meta), seg_offsets, E, H, max_rows,
                                                            make_ptrs(ret_ptrs, world));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_recv_expert_ids(const void* meta, int* counter, int capacity, int* expert_ids, int* n_out, int clear_counter,
                                  cudaStream_t s) {
  if (clear_counter) {
    if (capacity > 16384) return -1;    // one block only: the reset must follow every read of the counter
    recv_expert_ids_kernel<<<1, 1024, 0, s>>>(reinterpret_cast<const int4*>(meta), counter, capacity, expert_ids, n_out, 1);
  } else {
    recv_expert_ids_kernel<<<blocks_for(capacity, 256, 64), 256, 0, s>>>(reinterpret_cast<const int4*>(meta), counter, capacity,
                                                                        expert_ids, n_out, 0);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_sum_rows(const long long* src_ptrs, int world, void* out, long long numel, cudaStream_t s) {
  if (numel == 0) return 0;
  if (numel % 8) return -1;
  sum_rows_kernel<<<blocks_for(numel / 8, 256, 148 * 8), 256, 0, s>>>(make_ptrs(src_ptrs, world), world, reinterpret_cast<bf16*>(out),
                                                                    numel / 8);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_gather_rows(const long long* src_ptrs, int world, void* out, long long bytes_per_rank, cudaStream_t s) {
  if (bytes_per_rank == 0) return 0;
  if (bytes_per_rank % 16) return -1;
  gather_rows_kernel<<<blocks_for(bytes_per_rank / 16 * world, 256, 148 * 8), 256, 0, s>>>(make_ptrs(src_ptrs, world), world,
                                                                                         reinterpret_cast<uint4*>(out),
                                                                                         bytes_per_rank / 16);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_stats_merge(const long long* stats_ptrs, int world, long long R, float* logp, float* ent, float* lse, cudaStream_t s) {
  if (R == 0) return 0;
  stats_merge_kernel<<<static_cast<unsigned>((R + 255) / 256), 256, 0, s>>>(make_ptrs(stats_ptrs, world), world, R, logp, ent, lse);
  return static_cast<int>(cudaGetLastError());
}
