// Bindings: router top-k and MoE token permutation.
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

// logits fp32 [T,E] → (weights fp32 [T,K], idx int32 [T,K], probs fp32 [T,E])
std::vector<at::Tensor> router_topk(const at::Tensor& logits, int64_t K, bool normalize, bool want_probs) {
  c10::cuda::CUDAGuard g(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  auto w = at::empty({T, K}, logits.options());
  auto idx = at::empty({T, K}, logits.options().dtype(at::kInt));
  at::Tensor probs;
  if (want_probs) probs = at::empty({T, E}, logits.options());
  check(mb_router_topk(logits.data_ptr<float>(), want_probs ? probs.data_ptr<float>() : nullptr, w.data_ptr<float>(),
                       idx.data_ptr<int>(), T, E, K, normalize, cur_stream()),
        "mb_router_topk");
  return {w, idx, probs};
}

// idx int32 [n] global expert ids → seg_offsets [E+1], tile_expert [max_rows/pad], row_src [max_rows], dst_row [n]
std::vector<at::Tensor> moe_align(const at::Tensor& idx, int64_t E, int64_t expert_offset, int64_t max_rows,
                                  const c10::optional<at::Tensor>& n_dev, int64_t pad) {
  c10::cuda::CUDAGuard g(idx.device());
  const int64_t n = idx.numel();
  const int* n_ptr = n_dev.has_value() && n_dev->defined() ? n_dev->data_ptr<int>() : nullptr;
  auto opt = idx.options().dtype(at::kInt);
  auto seg = at::empty({E + 1}, opt);
  TORCH_CHECK(pad > 0 && max_rows % pad == 0, "moe_align: max_rows must be a multiple of pad");
  auto tile = at::empty({max_rows / pad}, opt);
  auto row_src = at::empty({max_rows}, opt);
  auto dst_row = at::empty({n}, opt);
  check(mb_moe_align_pad(idx.data_ptr<int>(), n, n_ptr, E, expert_offset, seg.data_ptr<int>(), tile.data_ptr<int>(),
                         row_src.data_ptr<int>(), dst_row.data_ptr<int>(), max_rows, pad, cur_stream()),
        "mb_moe_align");
  return {seg, tile, row_src, dst_row};
}

void moe_gather(const at::Tensor& x, at::Tensor& x_perm, const at::Tensor& row_src, const at::Tensor& seg, int64_t k) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_moe_gather(x.data_ptr(), x_perm.data_ptr(), row_src.data_ptr<int>(), seg.data_ptr<int>(), seg.numel() - 1, k, x.size(-1),
                      x_perm.size(0), cur_stream()),
        "mb_moe_gather");
}

void moe_combine(const at::Tensor& y_perm, const c10::optional<at::Tensor>& w, const at::Tensor& dst_row, at::Tensor& out, int64_t k,
                 bool identity_rows) {
  c10::cuda::CUDAGuard g(out.device());
  check(mb_moe_combine(y_perm.data_ptr(), w.has_value() && w->defined() ? w->data_ptr<float>() : nullptr, dst_row.data_ptr<int>(),
                       out.data_ptr(), out.size(0), k, out.size(-1), identity_rows ? 1 : 0, cur_stream()),
        "mb_moe_combine");
}

void moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y_perm, const at::Tensor& w, const at::Tensor& row_src,
                     const at::Tensor& seg, at::Tensor& dy_perm, const c10::optional<at::Tensor>& dw, int64_t k) {
  c10::cuda::CUDAGuard g(dout.device());
  check(mb_moe_combine_bwd(dout.data_ptr(), y_perm.data_ptr(), w.data_ptr<float>(), row_src.data_ptr<int>(), seg.data_ptr<int>(),
                           seg.numel() - 1, dy_perm.data_ptr(), dw.has_value() && dw->defined() ? dw->data_ptr<float>() : nullptr, k,
                           dout.size(-1), dy_perm.size(0), cur_stream()),
        "mb_moe_combine_bwd");
}

}  // namespace

void register_moe(pybind11::module& m) {
  m.def("router_topk", &router_topk);
  m.def("moe_align", &moe_align, py::arg("idx"), py::arg("E"), py::arg("expert_offset"), py::arg("max_rows"), py::arg("n_dev"),
        py::arg("pad") = 128);
  m.def("moe_gather", &moe_gather);
  m.def("moe_combine", &moe_combine, pybind11::arg("y_perm"), pybind11::arg("w"), pybind11::arg("dst_row"), pybind11::arg("out"),
        pybind11::arg("k"), pybind11::arg("identity_rows") = false);
  m.def("moe_combine_bwd", &moe_combine_bwd);
}
