// Sparse attention over a per-query index list (forward).  One warp per (query token, query head):
//   for every listed key row j ≥ 0:  s = scale · q·k[j];  online softmax;  acc += p · v[j]
// q [T, H, D], k [Tkv, Hk, D], v [Tkv, Hk, Dv] bf16 (H a multiple of Hk; Hk = 1 for a shared latent), indices int32
// [T, K] with −1 padding, optional per-head sink logit added to the softmax denominator.  Each lane keeps D/32 elements of
// q and Dv/32 of the accumulator in registers; a key costs one 5-step warp reduction.  The kernel is gather-bound
// (K·(D+Dv)·2 bytes per (query, kv head)); heads of one kv group run in the same CTA so the gathered rows hit in L1/L2.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kMaxDPerLane = 18;    // D ≤ 576
constexpr int kMaxDvPerLane = 16;   // Dv ≤ 512

__global__ void __launch_bounds__(256) sparse_attn_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                              const int* __restrict__ indices, const float* __restrict__ sink,
                                                              bf16* __restrict__ out, float* __restrict__ lse, long long T, int H, int Hk,
                                                              int D, int Dv, int K, long long Tkv, float scale) {
  const long long w = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const long long t = w / H;
  const int h = static_cast<int>(w % H);
  const int hk = h / (H / Hk);
  const int dpl = D / 32, dvpl = Dv / 32;
  float qr[kMaxDPerLane], acc[kMaxDvPerLane];
  for (int i = 0; i < dpl; ++i) qr[i] = __bfloat162float(q[(t * H + h) * D + i * 32 + lane]) * scale;
  for (int i = 0; i < dvpl; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (sink != nullptr) { m = sink[h]; l = 1.f; }
  const int* idx = indices + t * K;
  for (int j = 0; j < K; ++j) {
    const int row = idx[j];
    if (row < 0 || row >= Tkv) continue;                       // warp-uniform
    const bf16* kr = k + (static_cast<long long>(row) * Hk + hk) * D;
    float s = 0.f;
    for (int i = 0; i < dpl; ++i) s += qr[i] * __bfloat162float(kr[i * 32 + lane]);
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float m_new = fmaxf(m, s);
    const float corr = __expf(m - m_new), p = __expf(s - m_new);
    l = l * corr + p;
    const bf16* vr = v + (static_cast<long long>(row) * Hk + hk) * Dv;
    for (int i = 0; i < dvpl; ++i) acc[i] = acc[i] * corr + p * __bfloat162float(vr[i * 32 + lane]);
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int i = 0; i < dvpl; ++i) out[(t * H + h) * Dv + i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  if (lane == 0) lse[t * H + h] = l > 0.f ? m + logf(l) : -INFINITY;
}

}  // namespace
}  // namespace mb

extern "C" int mb_sparse_attention_fwd(const void* q, const void* k, const void* v, const int* indices, const float* sink, void* out,
                                       float* lse, long long T, int H, int Hk, int D, int Dv, int K, long long Tkv, float scale,
                                       cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 32 || Dv % 32 || D > 32 * mb::kMaxDPerLane || Dv > 32 * mb::kMaxDvPerLane || H % Hk) return -1;
  const long long warps = T * H;
  mb::sparse_attn_fwd_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(
      static_cast<const mb::bf16*>(q), static_cast<const mb::bf16*>(k), static_cast<const mb::bf16*>(v), indices, sink,
      static_cast<mb::bf16*>(out), lse, T, H, Hk, D, Dv, K, Tkv, scale);
  return static_cast<int>(cudaGetLastError());
}
