// Torch bindings: unwrap tensors to raw pointers and call the C launchers on the current CUDA stream.
// Shape/dtype checks live in python (`miles_b200/ops/cuda.py`); this file only marshals.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "launch.h"

namespace {

// The CUDA "last error" is per host thread and other code may have left one behind (it is not an error of ours):
// clear it before launching so that the launcher's own cudaGetLastError() reports only its launch.
inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  mb_count_launch(1);
  return at::cuda::getCurrentCUDAStream().stream();
}
inline const void* cptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline void* mptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline void check(int rc, const char* what) {
  if (rc == 0) return;
  char buf[256];
  snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc,
           rc > 0 && rc < 1000 ? cudaGetErrorString(static_cast<cudaError_t>(rc)) : "launcher");
  throw std::runtime_error(buf);
}

// One int32 per device, raised by kernels whose bounded waits ran out.
at::Tensor& error_flag_for(const at::Device& dev) {
  static std::vector<at::Tensor> flags(64);
  auto& f = flags[dev.index()];
  if (!f.defined()) f = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return f;
}

at::Tensor error_flag(const at::Tensor& like) { return error_flag_for(like.device()); }

void gemm(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
          int64_t ldc, bool a_mn, bool b_mn, bool accumulate, const c10::optional<at::Tensor>& bias, int64_t force_bn) {
  c10::cuda::CUDAGuard g(A.device());
  int* ef = error_flag_for(A.device()).data_ptr<int>();
  check(mb_gemm_bf16(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, lda, ldb, ldc, a_mn, b_mn, C.scalar_type() == at::kFloat,
                     accumulate, cptr(bias), force_bn, ef, cur_stream()),
        "mb_gemm_bf16");
}

void gemm_splitk(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, int64_t M, int64_t N, int64_t K, int64_t ldc,
                 bool accumulate, const c10::optional<at::Tensor>& bias, int64_t split_k, at::Tensor& ws, at::Tensor& counters) {
  c10::cuda::CUDAGuard g(A.device());
  int* ef = error_flag_for(A.device()).data_ptr<int>();
  check(mb_gemm_bf16_splitk(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, K, K, ldc, C.scalar_type() == at::kFloat, accumulate,
                            cptr(bias), split_k, ws.data_ptr<float>(), counters.data_ptr<int>(), ef, cur_stream()),
        "mb_gemm_bf16_splitk");
}

// C[tokens, N] = X[tokens, K] · W[N, K]ᵀ with the weight rows on the 128-row MMA side (decode-sized token counts)
void gemm_small(const at::Tensor& X, const at::Tensor& W, at::Tensor& C, int64_t tokens, int64_t N, int64_t K, int64_t ldc,
                const c10::optional<at::Tensor>& bias, int64_t bt, int64_t split_k, const c10::optional<at::Tensor>& ws,
                const c10::optional<at::Tensor>& counters) {
  c10::cuda::CUDAGuard g(X.device());
  int* ef = error_flag_for(X.device()).data_ptr<int>();
  check(mb_gemm_small(X.data_ptr(), W.data_ptr(), C.data_ptr(), tokens, N, K, K, K, ldc, C.scalar_type() == at::kFloat, cptr(bias), bt,
                      split_k, ws.has_value() && ws->defined() ? ws->data_ptr<float>() : nullptr,
                      counters.has_value() && counters->defined() ? counters->data_ptr<int>() : nullptr, ef, cur_stream()),
        "mb_gemm_small");
}

// y[M, N] = norm?(x (+ residual)) · Wᵀ (+ bias) for M ≤ 16; two kernel launches are counted by the MoE variant below
void gemv(const at::Tensor& x, const c10::optional<at::Tensor>& residual, const c10::optional<at::Tensor>& norm_w, double eps,
          const at::Tensor& W, const c10::optional<at::Tensor>& bias, at::Tensor& y, const c10::optional<at::Tensor>& res_out,
          const c10::optional<at::Tensor>& xn_out, bool static_w) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t K = x.size(-1), M = x.numel() / K, N = W.size(0);
  check(mb_gemv(x.data_ptr(), cptr(residual), cptr(norm_w), eps, W.data_ptr(), cptr(bias), y.data_ptr(), y.stride(0),
                y.scalar_type() == at::kFloat, mptr(res_out), mptr(xn_out), M, N, K, static_w, cur_stream()),
        "mb_gemv");
}

void moe_gemv(const at::Tensor& x, const at::Tensor& w13, const at::Tensor& w2, const at::Tensor& topk_idx, const at::Tensor& topk_w,
              at::Tensor& act, at::Tensor& out, int64_t expert_offset) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t T = x.size(0), H = x.size(1), k = topk_idx.size(1), E = w13.size(0), F = w13.size(1) / 2;
  mb_count_launch(1);
  check(mb_moe_gemv(x.data_ptr(), w13.data_ptr(), w2.data_ptr(), topk_idx.data_ptr<int>(), topk_w.data_ptr<float>(), act.data_ptr(),
                    out.data_ptr(), T, k, E, expert_offset, H, F, cur_stream()),
        "mb_moe_gemv");
}

void gemm_small_grouped(const at::Tensor& X, const at::Tensor& W, at::Tensor& C, int64_t rows, int64_t N, int64_t K, int64_t E,
                        const at::Tensor& tile_expert, const c10::optional<at::Tensor>& used_rows, int64_t bt) {
  c10::cuda::CUDAGuard g(X.device());
  int* ef = error_flag_for(X.device()).data_ptr<int>();
  check(mb_gemm_small_grouped(X.data_ptr(), W.data_ptr(), C.data_ptr(), rows, N, K, E, tile_expert.data_ptr<int>(),
                              used_rows.has_value() && used_rows->defined() ? used_rows->data_ptr<int>() : nullptr, bt, ef, cur_stream()),
        "mb_gemm_small_grouped");
}

void gemm_grouped(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, int64_t M_pad, int64_t N, int64_t K, int64_t E,
                  const at::Tensor& tile_expert, bool b_mn, int64_t force_bn) {
  c10::cuda::CUDAGuard g(A.device());
  int* ef = error_flag_for(A.device()).data_ptr<int>();
  check(mb_gemm_bf16_grouped(A.data_ptr(), B.data_ptr(), C.data_ptr(), M_pad, N, K, E, tile_expert.data_ptr<int>(), b_mn,
                             C.scalar_type() == at::kFloat, force_bn, ef, cur_stream()),
        "mb_gemm_bf16_grouped");
}

void gemm_grouped_wgrad(const at::Tensor& dY, const at::Tensor& X, at::Tensor& dW, int64_t M_pad, int64_t N, int64_t K, int64_t E,
                        const at::Tensor& seg_offsets, bool accumulate, int64_t force_bn) {
  c10::cuda::CUDAGuard g(dY.device());
  int* ef = error_flag_for(dY.device()).data_ptr<int>();
  check(mb_gemm_bf16_grouped_wgrad(dY.data_ptr(), X.data_ptr(), dW.data_ptr(), M_pad, N, K, E, seg_offsets.data_ptr<int>(),
                                   dW.scalar_type() == at::kFloat, accumulate, force_bn, ef, cur_stream()),
        "mb_gemm_bf16_grouped_wgrad");
}

void rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& residual, const at::Tensor& w, at::Tensor& y,
                 const c10::optional<at::Tensor>& res_out, const c10::optional<at::Tensor>& rstd, double eps) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t H = x.size(-1), T = x.numel() / H;
  check(mb_rmsnorm_fwd(x.data_ptr(), cptr(residual), w.data_ptr(), y.data_ptr(), mptr(res_out),
                       rstd.has_value() ? rstd->data_ptr<float>() : nullptr, T, H, eps, cur_stream()),
        "mb_rmsnorm_fwd");
}

at::Tensor rmsnorm_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy, const c10::optional<at::Tensor>& dres,
                       const at::Tensor& rstd, at::Tensor& dx) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t H = x.size(-1), T = x.numel() / H;
  at::Tensor dw = at::empty({H}, w.options());
  if (T == 0) return dw.zero_();
  const int blocks = mb_rmsnorm_bwd_blocks(T);
  at::Tensor partial = at::empty({blocks, H}, x.options().dtype(at::kFloat));
  check(mb_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), cptr(dres), rstd.data_ptr<float>(), dx.data_ptr(),
                       partial.data_ptr<float>(), dw.data_ptr(), 0, T, H, cur_stream()),
        "mb_rmsnorm_bwd");
  return dw;
}

void swiglu_fwd(const at::Tensor& in, at::Tensor& out, const c10::optional<at::Tensor>& rows) {
  c10::cuda::CUDAGuard g(in.device());
  const int64_t F = out.size(-1), T = out.numel() / std::max<int64_t>(F, 1);
  check(mb_swiglu_fwd(in.data_ptr(), out.data_ptr(), T, F, rows.has_value() && rows->defined() ? rows->data_ptr<int>() : nullptr,
                      cur_stream()),
        "mb_swiglu_fwd");
}

void swiglu_bwd(const at::Tensor& in, const at::Tensor& dout, at::Tensor& din, const c10::optional<at::Tensor>& rows) {
  c10::cuda::CUDAGuard g(in.device());
  const int64_t F = dout.size(-1), T = dout.numel() / std::max<int64_t>(F, 1);
  check(mb_swiglu_bwd(in.data_ptr(), dout.data_ptr(), din.data_ptr(), T, F,
                      rows.has_value() && rows->defined() ? rows->data_ptr<int>() : nullptr, cur_stream()),
        "mb_swiglu_bwd");
}

void qk_norm_rope_fwd(const at::Tensor& q, const at::Tensor& k, const c10::optional<at::Tensor>& qw,
                      const c10::optional<at::Tensor>& kw, const at::Tensor& positions, at::Tensor& qo, at::Tensor& ko,
                      const c10::optional<at::Tensor>& q_rstd, const c10::optional<at::Tensor>& k_rstd, double theta, double eps) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), Hk = k.size(1), D = q.size(2);
  check(mb_qk_norm_rope_fwd(q.data_ptr(), k.data_ptr(), q.stride(0), k.stride(0), cptr(qw), cptr(kw), positions.data_ptr<int>(),
                            qo.data_ptr(), ko.data_ptr(), q_rstd.has_value() ? q_rstd->data_ptr<float>() : nullptr,
                            k_rstd.has_value() ? k_rstd->data_ptr<float>() : nullptr, T, Hq, Hk, D, theta, eps, cur_stream()),
        "mb_qk_norm_rope_fwd");
}

at::Tensor rope(const at::Tensor& x, const at::Tensor& positions, double theta, bool inverse) {
  c10::cuda::CUDAGuard g(x.device());
  auto y = at::empty({x.size(0), x.size(1), x.size(2)}, x.options());
  check(mb_rope(x.data_ptr(), y.data_ptr(), positions.data_ptr<int>(), x.size(0), x.size(1), x.size(2), x.stride(0), theta, inverse ? 1 : 0,
                cur_stream()),
        "mb_rope");
  return y;
}

void qk_norm_rope_cache(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& qw,
                        const c10::optional<at::Tensor>& kw, const at::Tensor& positions, at::Tensor& qo, at::Tensor& ko,
                        at::Tensor& kc, at::Tensor& vc, const at::Tensor& slots, double theta, double eps) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), Hk = k.size(1), D = q.size(2);
  check(mb_qk_norm_rope_cache(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), cptr(qw), cptr(kw),
                              positions.data_ptr<int>(), qo.data_ptr(), ko.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                              reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()), T, Hq, Hk, D, theta, eps, cur_stream()),
        "mb_qk_norm_rope_cache");
}

// returns dw (bf16 [D]) or an undefined tensor when w is absent
at::Tensor qk_norm_rope_bwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, const c10::optional<at::Tensor>& rstd,
                            const at::Tensor& dy, const at::Tensor& positions, at::Tensor& dx, double theta) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t T = x.size(0), Hn = x.size(1), D = x.size(2);
  at::Tensor dw, partial;
  float* pp = nullptr;
  void* dwp = nullptr;
  if (w.has_value() && w->defined()) {
    dw = at::zeros({D}, w->options());
    if (T > 0) {
      partial = at::empty({mb_qk_norm_rope_bwd_blocks(T, Hn), D}, x.options().dtype(at::kFloat));
      pp = partial.data_ptr<float>();
      dwp = dw.data_ptr();
    }
  }
  check(mb_qk_norm_rope_bwd(x.data_ptr(), x.stride(0), cptr(w), rstd.has_value() && rstd->defined() ? rstd->data_ptr<float>() : nullptr,
                            dy.data_ptr(), positions.data_ptr<int>(), dx.data_ptr(), dx.stride(0), pp, dwp, T, Hn, D, theta,
                            cur_stream()),
        "mb_qk_norm_rope_bwd");
  return dw;
}

void kv_cache_write(const at::Tensor& k, const at::Tensor& v, at::Tensor& kc, at::Tensor& vc, const at::Tensor& slots) {
  c10::cuda::CUDAGuard g(k.device());
  const int64_t T = k.size(0), row = k.size(1) * k.size(2);
  check(mb_kv_cache_write(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), kc.data_ptr(), vc.data_ptr(),
                          reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()), T, row, cur_stream()),
        "mb_kv_cache_write");
}

void adamw(at::Tensor& master, const at::Tensor& grad, at::Tensor& m, at::Tensor& v, const c10::optional<at::Tensor>& decay_mask,
           const c10::optional<at::Tensor>& scale, const c10::optional<at::Tensor>& param_out, double lr, double b1, double b2,
           double eps, double wd, int64_t step) {
  c10::cuda::CUDAGuard g(master.device());
  const bool out_bf16 = param_out.has_value() && param_out->defined() && param_out->scalar_type() == at::kBFloat16;
  check(mb_adamw(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                 decay_mask.has_value() && decay_mask->defined() ? decay_mask->data_ptr<float>() : nullptr,
                 scale.has_value() && scale->defined() ? scale->data_ptr<float>() : nullptr, mptr(param_out), out_bf16,
                 master.numel(), lr, b1, b2, eps, wd, step, cur_stream()),
        "mb_adamw");
}

}  // namespace

void register_more(pybind11::module& m);  // bindings_more.cpp: attention, MoE, sampling, quantisation, fabric

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("error_flag", &error_flag);
  m.def("set_pdl", [](bool on) { mb_set_pdl(on ? 1 : 0); });
  m.def("pdl_enabled", []() { return mb_pdl_enabled() != 0; });
  m.def("launch_count", []() { return static_cast<int64_t>(mb_launch_count()); });
  m.def("count_launches", [](int64_t n) { mb_count_launch(static_cast<int>(n)); });
  m.def("gemm", &gemm);
  m.def("gemm_splitk", &gemm_splitk);
  m.def("gemm_grouped", &gemm_grouped);
  m.def("gemm_small", &gemm_small);
  m.def("gemv", &gemv);
  m.def("moe_gemv", &moe_gemv);
  m.def("gemm_small_grouped", &gemm_small_grouped);
  m.def("gemm_grouped_wgrad", &gemm_grouped_wgrad);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope", &rope);
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("qk_norm_rope_cache", &qk_norm_rope_cache);
  m.def("kv_cache_write", &kv_cache_write);
  m.def("adamw", &adamw);
  register_more(m);
}
