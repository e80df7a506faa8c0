// Vocabulary-sized row kernels: fused sampling with log-prob, and the streaming statistics / gradient kernels of
// the log-prob head (log-sum-exp, target logit and Σ p·logit accumulated chunk by chunk over the vocabulary so the
// full [tokens, vocab] logits never exist).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"
#include "pdl.cuh"

namespace mb {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t step, uint64_t idx) {
  const uint64_t h = splitmix64(splitmix64(seed * 0x100000001B3ull + step) ^ (idx * 0xD6E8FEB86659FD93ull));
  return (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

struct MS {  // running max / scaled sum
  float m, s;
};
__device__ __forceinline__ MS ms_merge(MS a, MS b) {
  if (a.m == -INFINITY) return b;
  if (b.m == -INFINITY) return a;
  const float m = fmaxf(a.m, b.m);
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}

// One CTA per row.  logits fp32 [B, V]; inv_temp[B]; greedy[B] (bool as uint8); seeds[B].
// token = argmax(logit·inv_temp + Gumbel) (greedy: argmax logit); logprob = logit[token]·inv_temp − lse.
__global__ void __launch_bounds__(1024) sample_logprob_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                              const uint8_t* __restrict__ greedy, const long long* __restrict__ seeds,
                                                              long long step, long long* __restrict__ tokens,
                                                              float* __restrict__ logprobs, int V) {
  __shared__ float sh_m[32], sh_s[32], sh_best[32];
  __shared__ int sh_idx[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float* x = logits + static_cast<long long>(row) * V;
  const float it = 1.f / temperature[row];
  const bool gr = greedy[row] != 0;
  const uint64_t seed = static_cast<uint64_t>(seeds ? seeds[row] : row);
  MS ms{-INFINITY, 0.f};
  float best = -INFINITY;
  int best_i = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float z = x[i] * it;
    ms = ms_merge(ms, MS{z, 1.f});
    float score = z;
    if (!gr) score += -__logf(-__logf(uniform01(seed, static_cast<uint64_t>(step), static_cast<uint64_t>(i))));
    if (score > best) { best = score; best_i = i; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MS other{__shfl_xor_sync(0xffffffffu, ms.m, o), __shfl_xor_sync(0xffffffffu, ms.s, o)};
    ms = ms_merge(ms, other);
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  if (lane == 0) { sh_m[warp] = ms.m; sh_s[warp] = ms.s; sh_best[warp] = best; sh_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    ms = (lane < nw) ? MS{sh_m[lane], sh_s[lane]} : MS{-INFINITY, 0.f};
    best = (lane < nw) ? sh_best[lane] : -INFINITY;
    best_i = (lane < nw) ? sh_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MS other{__shfl_xor_sync(0xffffffffu, ms.m, o), __shfl_xor_sync(0xffffffffu, ms.s, o)};
      ms = ms_merge(ms, other);
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    if (lane == 0) {
      tokens[row] = best_i;
      logprobs[row] = x[best_i] * it - (ms.m + __logf(ms.s));
    }
  }
}

// The same for few rows: `parts` CTAs per row each take a slice of the vocabulary and leave (max, Σexp, best score, best
// index) in `ws`; the last CTA of a row to arrive (counter) merges the slices.  counters[row] is zero on entry and on exit.
__global__ void __launch_bounds__(256) sample_logprob_split_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                                   const uint8_t* __restrict__ greedy, const long long* __restrict__ seeds,
                                                                   long long step, long long* __restrict__ tokens,
                                                                   float* __restrict__ logprobs, int V, int parts, float4* __restrict__ ws,
                                                                   int* __restrict__ counters) {
  __shared__ float sh_m[8], sh_s[8], sh_best[8];
  __shared__ int sh_idx[8];
  __shared__ int sh_last;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x / parts, part = blockIdx.x % parts;
  const float* x = logits + static_cast<long long>(row) * V;
  const float it = 1.f / temperature[row];
  const bool gr = greedy[row] != 0;
  const uint64_t seed = static_cast<uint64_t>(seeds ? seeds[row] : row);
  const int per = (V + parts - 1) / parts;
  const int lo = part * per, hi = min(V, lo + per);
  MS ms{-INFINITY, 0.f};
  float best = -INFINITY;
  int best_i = 0x7fffffff;   // "no candidate": loses every tie; clamped into the vocabulary before it is used as an index
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    const float z = x[i] * it;
    ms = ms_merge(ms, MS{z, 1.f});
    float score = z;
    if (!gr) score += -__logf(-__logf(uniform01(seed, static_cast<uint64_t>(step), static_cast<uint64_t>(i))));
    if (score > best) { best = score; best_i = i; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto warp_merge = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MS other{__shfl_xor_sync(0xffffffffu, ms.m, o), __shfl_xor_sync(0xffffffffu, ms.s, o)};
      ms = ms_merge(ms, other);
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
  };
  warp_merge();
  if (lane == 0) { sh_m[warp] = ms.m; sh_s[warp] = ms.s; sh_best[warp] = best; sh_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    ms = (lane < 8) ? MS{sh_m[lane], sh_s[lane]} : MS{-INFINITY, 0.f};
    best = (lane < 8) ? sh_best[lane] : -INFINITY;
    best_i = (lane < 8) ? sh_idx[lane] : 0x7fffffff;
    warp_merge();
    if (lane == 0) {
      __stcg(&ws[row * parts + part], make_float4(ms.m, ms.s, best, __int_as_float(best_i)));
      __threadfence();
      sh_last = atomicAdd(&counters[row], 1) == parts - 1;
    }
  }
  __syncthreads();
  if (!sh_last || warp != 0) return;
  __threadfence();
  float4 v = lane < parts ? __ldcg(&ws[row * parts + lane]) : make_float4(-INFINITY, 0.f, -INFINITY, __int_as_float(0x7fffffff));
  ms = MS{v.x, v.y};
  best = v.z;
  best_i = __float_as_int(v.w);
  warp_merge();
  if (lane == 0) {
    // a row whose logits are all NaN has no candidate: report token 0 with a NaN log-prob instead of indexing out of range
    if (best_i < 0 || best_i >= V) best_i = 0;
    tokens[row] = best_i;
    logprobs[row] = x[best_i] * it - (ms.m + __logf(ms.s));
    counters[row] = 0;
  }
}

// Streaming statistics over one vocabulary chunk.  stats[r] = {m, s, e, t}:
//   m running max of z = logit·inv_temp, s = Σ exp(z − m), e = Σ exp(z − m)·z, t = z[target] (if in this chunk).
__global__ void __launch_bounds__(256) logit_stats_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                                                          float4* __restrict__ stats, int Vc, int v0, float inv_temp, int first) {
  __shared__ float sh[3][8];
  const long long r = blockIdx.x;
  const float* x = logits + r * ld;
  float m = -INFINITY, s = 0.f, e = 0.f;
  for (int i = threadIdx.x; i < Vc; i += 256) {
    const float z = x[i] * inv_temp;
    if (z > m) {
      const float a = __expf(m - z);   // m = −inf → a = 0
      s = s * a + 1.f;
      e = e * a + z;
      m = z;
    } else {
      const float p = __expf(z - m);
      s += p;
      e += p * z;
    }
  }
  // merge across the block
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o), oe = __shfl_xor_sync(0xffffffffu, e, o);
    const float nm = fmaxf(m, om);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm), b = (om == -INFINITY) ? 0.f : __expf(om - nm);
    s = s * a + os * b;
    e = e * a + oe * b;
    m = nm;
  }
  if (lane == 0) { sh[0][warp] = m; sh[1][warp] = s; sh[2][warp] = e; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = -INFINITY, S = 0.f, E = 0.f;
    for (int w = 0; w < 8; ++w) {
      const float om = sh[0][w];
      const float nm = fmaxf(M, om);
      const float a = (M == -INFINITY) ? 0.f : __expf(M - nm), b = (om == -INFINITY) ? 0.f : __expf(om - nm);
      S = S * a + sh[1][w] * b;
      E = E * a + sh[2][w] * b;
      M = nm;
    }
    float4 st = first ? make_float4(-INFINITY, 0.f, 0.f, 0.f) : stats[r];
    const float nm = fmaxf(st.x, M);
    const float a = (st.x == -INFINITY) ? 0.f : __expf(st.x - nm), b = (M == -INFINITY) ? 0.f : __expf(M - nm);
    st.y = st.y * a + S * b;
    st.z = st.z * a + E * b;
    st.x = nm;
    const long long tg = targets[r] - v0;
    if (tg >= 0 && tg < Vc) st.w = x[tg] * inv_temp;
    stats[r] = st;
  }
}

// stats → logp = t − lse, entropy = lse − e/s, lse
__global__ void logit_stats_finish_kernel(const float4* __restrict__ stats, float* __restrict__ logp, float* __restrict__ ent,
                                          float* __restrict__ lse, long long R) {
  const long long r = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (r >= R) return;
  const float4 st = stats[r];
  const float l = st.x + __logf(st.y);
  logp[r] = st.w - l;
  if (ent != nullptr) ent[r] = l - st.z / st.y;
  if (lse != nullptr) lse[r] = l;
}

// dlogits chunk (bf16) for the backward of (logp, entropy):
//   d z_j = g_lp·(1[j = target] − p_j) − g_ent·p_j·(z_j − (lse − H)),  d logit = d z · inv_temp,  p_j = exp(z_j − lse)
__global__ void __launch_bounds__(256) logit_grad_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                                                         const float* __restrict__ lse, const float* __restrict__ ent,
                                                         const float* __restrict__ g_lp, const float* __restrict__ g_ent,
                                                         __nv_bfloat16* __restrict__ dlogits, long long ldd, int Vc, int v0,
                                                         float inv_temp) {
  const long long r = blockIdx.y;
  const float* x = logits + r * ld;
  const float l = lse[r];
  const float glp = g_lp ? g_lp[r] : 0.f;
  const float ge = g_ent ? g_ent[r] : 0.f;
  const float mean_z = (g_ent != nullptr) ? (l - ent[r]) : 0.f;
  const long long tg = targets[r] - v0;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < Vc; i += gridDim.x * 256) {
    const float z = x[i] * inv_temp;
    const float p = __expf(z - l);
    float d = -glp * p - ge * p * (z - mean_z);
    if (i == tg) d += glp;
    dlogits[r * ldd + i] = __float2bfloat16(d * inv_temp);
  }
}

}  // namespace mb

namespace mb {
// Hand-over between two decode steps of one host round trip, one thread per row: record the step's outputs, feed the
// sampled token back, advance position and length of live rows (length 0 = padding row), look the new cache slot up in
// the block table, advance the random seed.
__global__ void decode_advance_kernel(const long long* __restrict__ o_tok, const float* __restrict__ o_lp, const int* __restrict__ o_routed,
                                      long long* __restrict__ h_tok, float* __restrict__ h_lp, int* __restrict__ h_routed,
                                      int routed_per_row, int* __restrict__ tok, int* __restrict__ pos, int* __restrict__ len,
                                      const int* __restrict__ block_table, int max_blocks, int block_size,
                                      long long* __restrict__ slot, long long* __restrict__ seed, int B, int vocab,
                                      int* __restrict__ error_flag) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= B) return;
  long long t = o_tok[r];
  h_tok[r] = t;                 // the host sees what was sampled, in range or not, and fails the request with its context
  if (t < 0 || t >= vocab) {    // a non-finite hidden state upstream: never feed such an id to the next step's embedding lookup
    if (len[r] > 0 && error_flag != nullptr) atomicCAS(error_flag, 0, 71);
    t = 0;
  }
  h_lp[r] = o_lp[r];
  if (h_routed != nullptr)
    for (int i = 0; i < routed_per_row; ++i) h_routed[static_cast<long long>(r) * routed_per_row + i] = o_routed[static_cast<long long>(r) * routed_per_row + i];
  tok[r] = static_cast<int>(t);
  if (len[r] > 0) {
    const int p = pos[r] + 1;
    pos[r] = p;
    len[r] += 1;
    const int b = min(p / block_size, max_blocks - 1);
    slot[r] = static_cast<long long>(block_table[static_cast<long long>(r) * max_blocks + b]) * block_size + p % block_size;
  } else {
    slot[r] = -1;
  }
  seed[r] = (seed[r] + 1) & 0x7FFFFFFFFFFFFFFFll;
}
}  // namespace mb

using namespace mb;

extern "C" int mb_decode_advance(const long long* o_tok, const float* o_lp, const int* o_routed, long long* h_tok, float* h_lp,
                                 int* h_routed, int routed_per_row, int* tok, int* pos, int* len, const int* block_table, int max_blocks,
                                 int block_size, long long* slot, long long* seed, int B, int vocab, int* error_flag, cudaStream_t s) {
  if (B == 0) return 0;
  return static_cast<int>(launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, o_tok, o_lp, o_routed, h_tok, h_lp,
                                     h_routed, routed_per_row, tok, pos, len, block_table, max_blocks, block_size, slot, seed, B, vocab,
                                     error_flag));
}

extern "C" int mb_sample_logprob(const float* logits, const float* temperature, const uint8_t* greedy, const long long* seeds,
                                 long long step, long long* tokens, float* logprobs, int B, int V, cudaStream_t s) {
  if (B == 0) return 0;
  return static_cast<int>(launch_pdl(sample_logprob_kernel, dim3(B), dim3(1024), 0, s, logits, temperature, greedy, seeds, step, tokens,
                                     logprobs, V));
}

// parts CTAs per row (2…32); ws: 4·B·parts floats; counters: B ints, zero on entry (and again on exit)
extern "C" int mb_sample_logprob_split(const float* logits, const float* temperature, const uint8_t* greedy, const long long* seeds,
                                       long long step, long long* tokens, float* logprobs, int B, int V, int parts, float* ws,
                                       int* counters, cudaStream_t s) {
  if (B == 0) return 0;
  if (parts < 1 || parts > 32) return -1;
  return static_cast<int>(launch_pdl(sample_logprob_split_kernel, dim3(B * parts), dim3(256), 0, s, logits, temperature, greedy, seeds, step,
                                     tokens, logprobs, V, parts, reinterpret_cast<float4*>(ws), counters));
}

extern "C" int mb_logit_stats(const float* logits, long long ld, const long long* targets, float* stats, long long R, int Vc, int v0,
                              float inv_temp, int first, cudaStream_t s) {
  if (R == 0) return 0;
  logit_stats_kernel<<<static_cast<unsigned>(R), 256, 0, s>>>(logits, ld, targets, reinterpret_cast<float4*>(stats), Vc, v0, inv_temp, first);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_logit_stats_finish(const float* stats, float* logp, float* ent, float* lse, long long R, cudaStream_t s) {
  if (R == 0) return 0;
  logit_stats_finish_kernel<<<static_cast<unsigned>((R + 255) / 256), 256, 0, s>>>(reinterpret_cast<const float4*>(stats), logp, ent, lse, R);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mb_logit_grad(const float* logits, long long ld, const long long* targets, const float* lse, const float* ent,
                             const float* g_lp, const float* g_ent, void* dlogits, long long ldd, long long R, int Vc, int v0,
                             float inv_temp, cudaStream_t s) {
  if (R == 0) return 0;
  dim3 grid((Vc + 1023) / 1024, static_cast<unsigned>(R));
  if (R > 65535) return -1;
  logit_grad_kernel<<<grid, 256, 0, s>>>(logits, ld, targets, lse, ent, g_lp, g_ent, reinterpret_cast<__nv_bfloat16*>(dlogits), ldd, Vc,
                                         v0, inv_temp);
  return static_cast<int>(cudaGetLastError());
}
