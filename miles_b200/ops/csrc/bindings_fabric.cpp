// Bindings: symmetric (IPC-shared) device buffers and the peer-memory kernels of comm.cu.
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
inline void cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return;
  char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  throw std::runtime_error(buf);
}
inline const long long* lptr(const at::Tensor& t) { return reinterpret_cast<const long long*>(t.data_ptr<int64_t>()); }

at::Tensor wrap(void* ptr, int64_t nbytes, int device) {
  // memory is owned by the fabric for the life of the process (peers hold mappings of it), hence the empty deleter
  return at::from_blob(ptr, {nbytes}, [](void*) {}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
}

// cudaMalloc'd, zero-filled buffer + its IPC handle.  Plain cudaMalloc (not the caching allocator) so that the handle
// names exactly this allocation.
std::pair<at::Tensor, pybind11::bytes> fabric_alloc(int64_t nbytes, int64_t device) {
  c10::cuda::CUDAGuard g(static_cast<c10::DeviceIndex>(device));
  void* ptr = nullptr;
  cuda_ok(cudaMalloc(&ptr, static_cast<size_t>(nbytes)), "cudaMalloc(symmetric buffer)");
  cuda_ok(cudaMemset(ptr, 0, static_cast<size_t>(nbytes)), "cudaMemset(symmetric buffer)");
  cudaIpcMemHandle_t h;
  cuda_ok(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
  cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  return {wrap(ptr, nbytes, device), pybind11::bytes(reinterpret_cast<const char*>(&h), sizeof(h))};
}

// Map a peer's buffer into this process; the tensor lives on the *local* device index for bookkeeping but its
// memory is the peer's.  It is only ever handed to the kernels of comm.cu / the fused GEMMs, never to library kernels.
at::Tensor fabric_open(const std::string& handle, int64_t nbytes, int64_t device) {
  c10::cuda::CUDAGuard g(static_cast<c10::DeviceIndex>(device));
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle.data(), sizeof(h));
  void* ptr = nullptr;
  cuda_ok(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return wrap(ptr, nbytes, device);
}

void barrier(const at::Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t channel, at::Tensor& epochs, at::Tensor& err) {
  c10::cuda::CUDAGuard g(epochs.device());
  check(mb_barrier(lptr(flag_ptrs), rank, world, channel, epochs.data_ptr<int>(), err.data_ptr<int>(), cur_stream()), "mb_barrier");
}

void ar_add_rmsnorm(const at::Tensor& partial_ptrs, int64_t world, const c10::optional<at::Tensor>& residual, const at::Tensor& w,
                    at::Tensor& y, const c10::optional<at::Tensor>& res_out, double eps) {
  c10::cuda::CUDAGuard g(y.device());
  const int64_t H = y.size(-1), T = y.numel() / H;
  check(mb_ar_add_rmsnorm(lptr(partial_ptrs), world, residual.has_value() && residual->defined() ? residual->data_ptr() : nullptr,
                          w.data_ptr(), y.data_ptr(), res_out.has_value() && res_out->defined() ? res_out->data_ptr() : nullptr, T, H,
                          eps, cur_stream()),
        "mb_ar_add_rmsnorm");
}

void rs_reduce_sqnorm(const at::Tensor& grad_ptrs, int64_t world, int64_t rank, int64_t lo, int64_t hi,
                      const c10::optional<at::Tensor>& norm_weight, at::Tensor& sqnorm) {
  c10::cuda::CUDAGuard g(sqnorm.device());
  check(mb_rs_reduce_sqnorm(lptr(grad_ptrs), world, rank, lo, hi,
                            norm_weight.has_value() && norm_weight->defined() ? norm_weight->data_ptr<float>() : nullptr,
                            sqnorm.data_ptr<float>(), cur_stream()),
        "mb_rs_reduce_sqnorm");
}

void adam_allgather(at::Tensor& master, const at::Tensor& grad_shard, at::Tensor& m, at::Tensor& v,
                    const c10::optional<at::Tensor>& decay_mask, const c10::optional<at::Tensor>& sqnorm, double clip,
                    const at::Tensor& param_ptrs, int64_t world, int64_t lo, double lr, double b1, double b2, double eps, double wd,
                    int64_t step) {
  c10::cuda::CUDAGuard g(master.device());
  check(mb_adam_allgather(master.data_ptr<float>(), grad_shard.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                          decay_mask.has_value() && decay_mask->defined() ? decay_mask->data_ptr<float>() : nullptr,
                          sqnorm.has_value() && sqnorm->defined() ? sqnorm->data_ptr<float>() : nullptr, clip, lptr(param_ptrs), world,
                          lo, master.numel(), lr, b1, b2, eps, wd, step, cur_stream()),
        "mb_adam_allgather");
}

void moe_dispatch(const at::Tensor& x, const at::Tensor& topk_idx, int64_t k, int64_t e_local, int64_t rank,
                  const at::Tensor& recv_x_ptrs, const at::Tensor& recv_meta_ptrs, const at::Tensor& counter_ptrs, int64_t world,
                  int64_t capacity, at::Tensor& sent_row, at::Tensor& err) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_moe_dispatch(x.data_ptr(), topk_idx.data_ptr<int>(), topk_idx.numel(), k, x.size(-1), e_local, rank, lptr(recv_x_ptrs),
                        lptr(recv_meta_ptrs), lptr(counter_ptrs), world, capacity, sent_row.data_ptr<int>(), err.data_ptr<int>(),
                        cur_stream()),
        "mb_moe_dispatch");
}

void moe_dispatch_signal(const at::Tensor& x, const at::Tensor& topk_idx, int64_t k, int64_t e_local, int64_t rank,
                         const at::Tensor& recv_x_ptrs, const at::Tensor& recv_meta_ptrs, const at::Tensor& counter_ptrs, int64_t world,
                         int64_t capacity, at::Tensor& sent_row, at::Tensor& err, const at::Tensor& flag_ptrs, int64_t channel,
                         at::Tensor& epochs, at::Tensor& ticket) {
  c10::cuda::CUDAGuard g(x.device());
  check(mb_moe_dispatch_signal(x.data_ptr(), topk_idx.data_ptr<int>(), topk_idx.numel(), k, x.size(-1), e_local, rank, lptr(recv_x_ptrs),
                               lptr(recv_meta_ptrs), lptr(counter_ptrs), world, capacity, sent_row.data_ptr<int>(), err.data_ptr<int>(),
                               lptr(flag_ptrs), channel, epochs.data_ptr<int>(), ticket.data_ptr<int>(), cur_stream()),
        "mb_moe_dispatch_signal");
}

void moe_recv_align(const at::Tensor& meta, at::Tensor& counter, int64_t capacity, int64_t E, at::Tensor& seg, at::Tensor& tile,
                    at::Tensor& row_src, int64_t pad, const at::Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t channel,
                    const at::Tensor& epochs, at::Tensor& err) {
  c10::cuda::CUDAGuard g(meta.device());
  check(mb_moe_recv_align(meta.data_ptr(), counter.data_ptr<int>(), capacity, E, seg.data_ptr<int>(), tile.data_ptr<int>(),
                          row_src.data_ptr<int>(), row_src.numel(), pad, lptr(flag_ptrs), rank, world, channel, epochs.data_ptr<int>(),
                          err.data_ptr<int>(), cur_stream()),
        "mb_moe_recv_align");
}

void moe_return_signal(const at::Tensor& y_perm, const at::Tensor& row_src, const at::Tensor& meta, const at::Tensor& seg,
                       const at::Tensor& ret_ptrs, int64_t world, const at::Tensor& flag_ptrs, int64_t rank, int64_t channel,
                       at::Tensor& epochs, at::Tensor& ticket) {
  c10::cuda::CUDAGuard g(y_perm.device());
  check(mb_moe_return_signal(y_perm.data_ptr(), row_src.data_ptr<int>(), meta.data_ptr(), seg.data_ptr<int>(), seg.numel() - 1,
                             y_perm.size(-1), y_perm.size(0), lptr(ret_ptrs), world, lptr(flag_ptrs), rank, channel,
                             epochs.data_ptr<int>(), ticket.data_ptr<int>(), cur_stream()),
        "mb_moe_return_signal");
}

void moe_combine_wait(const at::Tensor& ret, const at::Tensor& w, const at::Tensor& sent_row, at::Tensor& out, int64_t k,
                      const at::Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t channel, const at::Tensor& epochs, at::Tensor& err) {
  c10::cuda::CUDAGuard g(out.device());
  check(mb_moe_combine_wait(ret.data_ptr(), w.data_ptr<float>(), sent_row.data_ptr<int>(), out.data_ptr(), out.size(0), k, out.size(-1),
                            lptr(flag_ptrs), rank, world, channel, epochs.data_ptr<int>(), err.data_ptr<int>(), cur_stream()),
        "mb_moe_combine_wait");
}

void moe_scatter_known(const at::Tensor& rows_in, bool src_by_pair, const at::Tensor& topk_idx, const at::Tensor& sent_row, int64_t k,
                       int64_t e_local, const at::Tensor& recv_x_ptrs, int64_t world) {
  c10::cuda::CUDAGuard g(rows_in.device());
  check(mb_moe_scatter_known(rows_in.data_ptr(), src_by_pair, topk_idx.data_ptr<int>(), sent_row.data_ptr<int>(), topk_idx.numel(), k,
                             rows_in.size(-1), e_local, lptr(recv_x_ptrs), world, cur_stream()),
        "mb_moe_scatter_known");
}

void moe_return(const at::Tensor& y_perm, const at::Tensor& row_src, const at::Tensor& meta, const at::Tensor& seg, const at::Tensor& ret_ptrs,
                int64_t world) {
  c10::cuda::CUDAGuard g(y_perm.device());
  check(mb_moe_return(y_perm.data_ptr(), row_src.data_ptr<int>(), meta.data_ptr(), seg.data_ptr<int>(), seg.numel() - 1, y_perm.size(-1),
                      y_perm.size(0), lptr(ret_ptrs), world, cur_stream()),
        "mb_moe_return");
}

void recv_expert_ids(const at::Tensor& meta, at::Tensor& counter, int64_t capacity, at::Tensor& expert_ids, at::Tensor& n_out,
                     bool clear_counter) {
  c10::cuda::CUDAGuard g(meta.device());
  check(mb_recv_expert_ids(meta.data_ptr(), counter.data_ptr<int>(), capacity, expert_ids.data_ptr<int>(), n_out.data_ptr<int>(),
                           clear_counter ? 1 : 0, cur_stream()),
        "mb_recv_expert_ids");
}

void stats_merge(const at::Tensor& stats_ptrs, int64_t world, at::Tensor& logp, const c10::optional<at::Tensor>& ent,
                 const c10::optional<at::Tensor>& lse) {
  c10::cuda::CUDAGuard g(logp.device());
  check(mb_stats_merge(lptr(stats_ptrs), world, logp.numel(), logp.data_ptr<float>(),
                       ent.has_value() && ent->defined() ? ent->data_ptr<float>() : nullptr,
                       lse.has_value() && lse->defined() ? lse->data_ptr<float>() : nullptr, cur_stream()),
        "mb_stats_merge");
}

void sum_rows(const at::Tensor& src_ptrs, int64_t world, at::Tensor& out) {
  c10::cuda::CUDAGuard g(out.device());
  check(mb_sum_rows(lptr(src_ptrs), world, out.data_ptr(), out.numel(), cur_stream()), "mb_sum_rows");
}

void gather_rows(const at::Tensor& src_ptrs, int64_t world, at::Tensor& out) {
  c10::cuda::CUDAGuard g(out.device());
  check(mb_gather_rows(lptr(src_ptrs), world, out.data_ptr(), out.numel() * out.element_size() / world, cur_stream()),
        "mb_gather_rows");
}

void ag_gemm(const at::Tensor& xg_ptrs, const at::Tensor& W, at::Tensor& Y, at::Tensor& block_counters, int64_t rows_per_rank,
             int64_t rank, int64_t world, const at::Tensor& flag_ptrs, int64_t channel, int64_t epoch, at::Tensor& err) {
  c10::cuda::CUDAGuard g(Y.device());
  TORCH_CHECK(block_counters.numel() * 128 >= rows_per_rank * world, "block_counters too small");
  check(mb_ag_gemm(lptr(xg_ptrs), W.data_ptr(), Y.data_ptr(), block_counters.data_ptr<int>(), rows_per_rank, W.size(0), W.size(1), rank,
                   world, lptr(flag_ptrs), channel, epoch, err.data_ptr<int>(), cur_stream()),
        "mb_ag_gemm");
}

// error flag address + peer wait limit for the kernels that talk to peers (0 keeps the current limit)
void fabric_configure(at::Tensor& err, int64_t wait_ns) {
  c10::cuda::CUDAGuard g(err.device());
  check(mb_comm_configure(err.data_ptr<int>(), static_cast<unsigned long long>(wait_ns)), "mb_comm_configure");
  check(mb_gemm_comm_configure(err.data_ptr<int>(), static_cast<unsigned long long>(wait_ns)), "mb_gemm_comm_configure");
}

void gemm_rs(const at::Tensor& X, const at::Tensor& W, const at::Tensor& partial_ptrs, at::Tensor& out, at::Tensor& counters,
             int64_t rank, int64_t world, const at::Tensor& flag_ptrs, int64_t channel, int64_t epoch, at::Tensor& err) {
  c10::cuda::CUDAGuard g(X.device());
  check(mb_gemm_rs(X.data_ptr(), W.data_ptr(), lptr(partial_ptrs), out.data_ptr(), counters.data_ptr<int>(), X.size(0), W.size(0),
                   X.size(1), rank, world, lptr(flag_ptrs), channel, epoch, err.data_ptr<int>(), cur_stream()),
        "mb_gemm_rs");
}

// one launch per bucket: table int64 [n,4] and prefix int64 [n+1] live on the device
void multi_copy(const at::Tensor& table, const at::Tensor& prefix, int64_t total_chunks) {
  c10::cuda::CUDAGuard g(table.device());
  check(mb_multi_copy(lptr(table), lptr(prefix), table.size(0), total_chunks, cur_stream()), "mb_multi_copy");
}

// rectangles {src, dst, rows, row_bytes, src_pitch, dst_pitch}: the resharding copy (dst may be a peer GPU's buffer)
void multi_copy2d(const at::Tensor& table, const at::Tensor& prefix, int64_t total_items, bool qdq) {
  c10::cuda::CUDAGuard g(table.device());
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 6, "multi_copy2d: table must be [n, 6]");
  check(mb_multi_copy2d(lptr(table), lptr(prefix), table.size(0), total_items, qdq ? 1 : 0, cur_stream()), "mb_multi_copy2d");
}

void multi_mxfp8(const at::Tensor& table, const at::Tensor& prefix, int64_t total_chunks, bool qdq) {
  c10::cuda::CUDAGuard g(table.device());
  check(mb_multi_mxfp8(lptr(table), lptr(prefix), table.size(0), total_chunks, qdq, cur_stream()), "mb_multi_mxfp8");
}

}  // namespace

void register_fabric(pybind11::module& m) {
  m.def("multi_copy", &multi_copy);
  m.def("multi_mxfp8", &multi_mxfp8);
  m.def("multi_copy2d", &multi_copy2d);
  m.def("ag_gemm", &ag_gemm);
  m.def("fabric_configure", &fabric_configure);
  m.def("gemm_rs", &gemm_rs);
  m.def("sum_rows", &sum_rows);
  m.def("gather_rows", &gather_rows);
  m.def("fabric_alloc", &fabric_alloc);
  m.def("fabric_open", &fabric_open);
  m.def("barrier", &barrier);
  m.def("ar_add_rmsnorm", &ar_add_rmsnorm);
  m.def("rs_reduce_sqnorm", &rs_reduce_sqnorm);
  m.def("adam_allgather", &adam_allgather);
  m.def("moe_dispatch", &moe_dispatch);
  m.def("moe_scatter_known", &moe_scatter_known);
  m.def("moe_dispatch_signal", &moe_dispatch_signal);
  m.def("moe_recv_align", &moe_recv_align);
  m.def("moe_return_signal", &moe_return_signal);
  m.def("moe_combine_wait", &moe_combine_wait);
  m.def("moe_return", &moe_return);
  m.def("recv_expert_ids", &recv_expert_ids, pybind11::arg("meta"), pybind11::arg("counter"), pybind11::arg("capacity"),
        pybind11::arg("expert_ids"), pybind11::arg("n_out"), pybind11::arg("clear_counter") = false);
  m.def("stats_merge", &stats_merge);
}
