// Bindings of extra.cu.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "launch.h"

namespace {

inline cudaStream_t cur_stream() {
  (void)cudaGetLastError();
  mb_count_launch(1);
  return at::cuda::getCurrentCUDAStream().stream();
}
inline void check(int rc, const char* what) {
  if (rc == 0) return;
  char buf[256];
  snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc,
           rc > 0 && rc < 1000 ? cudaGetErrorString(static_cast<cudaError_t>(rc)) : "launcher");
  throw std::runtime_error(buf);
}
inline bool is_f32(const at::Tensor& t) { return t.scalar_type() == at::kFloat; }

void grouped_rmsnorm(const at::Tensor& x, const at::Tensor& w, at::Tensor& out, at::Tensor& rstd, int64_t n, double eps) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t T = x.size(0), C = x.size(1) / n;
  check(mb_grouped_rmsnorm(x.data_ptr(), is_f32(x), w.data_ptr<float>(), out.data_ptr<float>(), rstd.data_ptr<float>(), T, n, C, eps, cur_stream()),
        "mb_grouped_rmsnorm");
}

void short_conv(const at::Tensor& x, const at::Tensor& w, const at::Tensor& bos, at::Tensor& y) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_short_conv(x.data_ptr(), is_f32(x), w.data_ptr<float>(), bos.data_ptr<int>(), y.data_ptr(), x.size(0), x.size(1), w.size(1), cur_stream()),
        "mb_short_conv");
}

void mhc_mix(const at::Tensor& x, const at::Tensor& res, const at::Tensor& h_res, const at::Tensor& h_post, at::Tensor& out, int64_t n) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_mhc_mix(x.data_ptr(), res.data_ptr(), h_res.data_ptr<float>(), h_post.data_ptr<float>(), out.data_ptr(), is_f32(x), x.size(0), n, x.size(1),
                   cur_stream()),
        "mb_mhc_mix");
}

void mhc_aggregate(const at::Tensor& x, const at::Tensor& pre, at::Tensor& out, int64_t n) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_mhc_aggregate(x.data_ptr(), is_f32(x), pre.data_ptr<float>(), out.data_ptr<float>(), x.size(0), n, x.size(1) / n, cur_stream()),
        "mb_mhc_aggregate");
}

void hc_combine(const at::Tensor& res, const at::Tensor& y, const at::Tensor& h_post, at::Tensor& out, int64_t n) {
  c10::cuda::CUDAGuard g(res.device());
  check(mb_hc_combine(res.data_ptr(), y.data_ptr(), h_post.data_ptr<float>(), out.data_ptr(), is_f32(res), res.size(0), n, y.size(1), cur_stream()),
        "mb_hc_combine");
}

void act_quant_1x128(const at::Tensor& x, const c10::optional<at::Tensor>& q, const c10::optional<at::Tensor>& qdq, at::Tensor& scales,
                     bool round_scale) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_act_quant_1x128(x.data_ptr(), q.has_value() ? q->data_ptr() : nullptr, qdq.has_value() ? qdq->data_ptr() : nullptr,
                           scales.data_ptr<float>(), x.size(0), x.size(1), round_scale, cur_stream()),
        "mb_act_quant_1x128");
}

void fp8_dequant(const at::Tensor& q, const c10::optional<at::Tensor>& scale_inv, const c10::optional<at::Tensor>& e8m0, at::Tensor& out) {
  c10::cuda::CUDAGuard g(q.device());
  check(mb_fp8_dequant(q.data_ptr(), scale_inv.has_value() ? scale_inv->data_ptr<float>() : nullptr,
                       e8m0.has_value() ? e8m0->data_ptr() : nullptr, out.data_ptr(), q.size(0), q.size(1), cur_stream()),
        "mb_fp8_dequant");
}

// `table` is a pinned CPU tensor [rows, width]; the kernel reads it through its device alias
void gather_rows_host(const at::Tensor& table, const at::Tensor& ids, at::Tensor& out) {
  c10::cuda::CUDAGuard g(out.device());
  TORCH_CHECK(table.is_pinned(), "gather_rows_host: the table must live in pinned host memory");
  void* dev = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&dev, table.data_ptr(), 0);
  if (e != cudaSuccess) check(static_cast<int>(e), "cudaHostGetDevicePointer");
  check(mb_gather_rows_host(dev, reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), out.data_ptr(), ids.numel(),
                            table.size(1) * table.element_size(), table.size(0), cur_stream()),
        "mb_gather_rows_host");
}

void sparse_attention_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& indices,
                          const c10::optional<at::Tensor>& sink, at::Tensor& out, at::Tensor& lse, double scale) {
  c10::cuda::CUDAGuard g(q.device());
  check(mb_sparse_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), indices.data_ptr<int>(),
                                sink.has_value() ? sink->data_ptr<float>() : nullptr, out.data_ptr(), lse.data_ptr<float>(), q.size(0), q.size(1),
                                k.size(1), q.size(2), v.size(2), indices.size(1), k.size(0), scale, cur_stream()),
        "mb_sparse_attention_fwd");
}

void gemm_mxfp8(const at::Tensor& A, const at::Tensor& sa, const at::Tensor& B, const at::Tensor& sb, at::Tensor& C, at::Tensor& err) {
  c10::cuda::CUDAGuard g(A.device());
  check(mb_gemm_mxfp8(A.data_ptr(), sa.data_ptr(), B.data_ptr(), sb.data_ptr(), C.data_ptr(), A.size(0), B.size(0), A.size(1), C.stride(0),
                      err.data_ptr<int>(), cur_stream()),
        "mb_gemm_mxfp8");
}

// A [M_pad, K] / sa: expert-sorted rows (segments padded to 128); B [E, N, K] / sb [E, N, K/32]; tile_expert int32 [M_pad/128]
void gemm_mxfp8_grouped(const at::Tensor& A, const at::Tensor& sa, const at::Tensor& B, const at::Tensor& sb, at::Tensor& C,
                        const at::Tensor& tile_expert, at::Tensor& err) {
  c10::cuda::CUDAGuard g(A.device());
  check(mb_gemm_mxfp8_grouped(A.data_ptr(), sa.data_ptr(), B.data_ptr(), sb.data_ptr(), C.data_ptr(), A.size(0), B.size(1), A.size(1),
                              B.size(0), tile_expert.data_ptr<int>(), C.stride(0), err.data_ptr<int>(), cur_stream()),
        "mb_gemm_mxfp8_grouped");
}

}  // namespace

void register_extra(pybind11::module& m) {
  m.def("gemm_mxfp8", &gemm_mxfp8);
  m.def("gemm_mxfp8_grouped", &gemm_mxfp8_grouped);
  m.def("sparse_attention_fwd", &sparse_attention_fwd);
  m.def("grouped_rmsnorm", &grouped_rmsnorm);
  m.def("short_conv", &short_conv);
  m.def("mhc_mix", &mhc_mix);
  m.def("mhc_aggregate", &mhc_aggregate);
  m.def("hc_combine", &hc_combine);
  m.def("act_quant_1x128", &act_quant_1x128);
  m.def("fp8_dequant", &fp8_dequant);
  m.def("gather_rows_host", &gather_rows_host);
}
