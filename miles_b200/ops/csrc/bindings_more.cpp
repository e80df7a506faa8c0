// Bindings for attention, MoE routing/permutation, sampling, log-prob, quantisation and the fabric kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <execinfo.h>
#include <signal.h>
#include <torch/extension.h>
#include <unistd.h>

#include "launch.h"

namespace {

inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  mb_count_launch(1);  // drop a stale per-thread error left by other code
  return at::cuda::getCurrentCUDAStream().stream();
}
inline const void* cptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline void* mptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline float* fptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr<float>() : nullptr; }
inline void check(int rc, const char* what) {
  if (rc == 0) return;
  char buf[256];
  snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc,
           rc > 0 && rc < 1000 ? cudaGetErrorString(static_cast<cudaError_t>(rc)) : "launcher");
  throw std::runtime_error(buf);
}

void crash_handler(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char msg[] = "\n*** fatal signal: native backtrace ***\n";
  (void)!write(2, msg, sizeof(msg) - 1);
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
// Print a native backtrace on SIGSEGV / SIGABRT / SIGBUS (debugging aid for crashes inside native code).
void install_crash_handler() {
  signal(SIGSEGV, crash_handler);
  signal(SIGABRT, crash_handler);
  signal(SIGBUS, crash_handler);
}

// ---- attention ---------------------------------------------------------------------------------
void flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, const c10::optional<at::Tensor>& lse,
               const at::Tensor& cu_seqlens, int64_t max_seqlen, double scale, bool causal) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  check(mb_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), fptr(lse), cu_seqlens.data_ptr<int>(),
                     cu_seqlens.numel() - 1, max_seqlen, T, q.stride(0), k.stride(0), v.stride(0), Hq, Hkv, D, scale, causal,
                     cur_stream()),
        "mb_flash_fwd");
}

void flash_fwd_tc(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, const c10::optional<at::Tensor>& lse,
                  const at::Tensor& cu_seqlens, int64_t max_seqlen, double scale, bool causal, at::Tensor& err,
                  const c10::optional<at::Tensor>& cu_seqlens_k) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), Hkv = k.size(1);
  const int* cuk = cu_seqlens_k.has_value() ? cu_seqlens_k->data_ptr<int>() : nullptr;
  check(mb_flash_fwd_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), fptr(lse), cu_seqlens.data_ptr<int>(),
                        cu_seqlens.numel() - 1, max_seqlen, T, q.stride(0), k.stride(0), v.stride(0), Hq, Hkv, scale, causal,
                        err.data_ptr<int>(), cuk, static_cast<int>(k.size(0)), cur_stream()),
        "mb_flash_fwd_tc");
}

void flash_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o, const at::Tensor& dout,
               const at::Tensor& lse, at::Tensor& delta, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv, const at::Tensor& cu_seqlens,
               int64_t max_seqlen, double scale, bool causal) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  check(mb_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                     delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_seqlens.data_ptr<int>(),
                     cu_seqlens.numel() - 1, max_seqlen, T, q.stride(0), k.stride(0), v.stride(0), Hq, Hkv, D, scale, causal,
                     cur_stream()),
        "mb_flash_bwd");
}

// tcgen05 backward (head_dim 128): delta pre-pass + dK/dV kernel + dQ kernel
void flash_bwd_tc(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o, const at::Tensor& dout,
                  const at::Tensor& lse, at::Tensor& delta, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv, const at::Tensor& cu_seqlens,
                  int64_t max_seqlen, double scale, bool causal, at::Tensor& err) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  TORCH_CHECK(D == 128, "flash_bwd_tc serves head_dim 128");
  check(mb_attn_delta(o.data_ptr(), dout.data_ptr(), delta.data_ptr<float>(), T, Hq, D, cur_stream()), "mb_attn_delta");
  mb_count_launch(2);
  check(mb_flash_bwd_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_seqlens.data_ptr<int>(), cu_seqlens.numel() - 1, max_seqlen, T,
                        q.stride(0), k.stride(0), v.stride(0), Hq, Hkv, scale, causal, err.data_ptr<int>(), cur_stream()),
        "mb_flash_bwd_tc");
}

void paged_decode(const at::Tensor& q, const at::Tensor& kc, const at::Tensor& vc, const at::Tensor& block_table,
                  const at::Tensor& seq_lens, at::Tensor& out, at::Tensor& part_o, at::Tensor& part_ml, double scale,
                  int64_t num_splits) {
  c10::cuda::CUDAGuard g(q.device());
  const int64_t B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = kc.size(2), bs = kc.size(1);
  check(mb_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), block_table.data_ptr<int>(), seq_lens.data_ptr<int>(),
                        out.data_ptr(), part_o.data_ptr<float>(), part_ml.data_ptr<float>(), B, block_table.size(1), bs, Hq, Hkv, D,
                        scale, num_splits, cur_stream()),
        "mb_paged_decode");
}

}  // namespace

void register_moe(pybind11::module& m);    // bindings_moe.cpp
void register_misc(pybind11::module& m);   // bindings_misc.cpp
void register_fabric(pybind11::module& m); // bindings_fabric.cpp
void register_extra(pybind11::module& m);  // bindings_extra.cpp

void register_more(pybind11::module& m) {
  m.def("install_crash_handler", &install_crash_handler);
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_fwd_tc", &flash_fwd_tc);
  m.def("flash_fwd_tc_ctas_per_sm", []() { return mb_flash_fwd_tc_ctas_per_sm(); });
  m.def("flash_bwd", &flash_bwd);
  m.def("flash_bwd_tc", &flash_bwd_tc);
  m.def("paged_decode", &paged_decode);
  register_moe(m);
  register_misc(m);
  register_fabric(m);
  register_extra(m);
}
