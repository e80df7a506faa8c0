// Bindings: sampling, log-prob statistics, quantisation.
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
inline float* fptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr<float>() : nullptr; }
inline void check(int rc, const char* what) {
  if (rc == 0) return;
  char buf[256];
  snprintf(buf, sizeof(buf), "%s failed with code %d (%s)", what, rc,
           rc > 0 && rc < 1000 ? cudaGetErrorString(static_cast<cudaError_t>(rc)) : "launcher");
  throw std::runtime_error(buf);
}

// device-side hand-over between two decode steps of one host round trip (see decode_advance_kernel)
void decode_advance(const at::Tensor& o_tok, const at::Tensor& o_lp, const c10::optional<at::Tensor>& o_routed, at::Tensor& h_tok,
                    at::Tensor& h_lp, const c10::optional<at::Tensor>& h_routed, at::Tensor& tok, at::Tensor& pos, at::Tensor& len,
                    const at::Tensor& block_table, int64_t block_size, at::Tensor& slot, at::Tensor& seed, int64_t vocab,
                    at::Tensor& error_flag) {
  c10::cuda::CUDAGuard g(o_tok.device());
  const int64_t B = tok.numel();
  const bool rec = o_routed.has_value() && o_routed->defined() && h_routed.has_value() && h_routed->defined();
  const int64_t per = rec ? o_routed->numel() / std::max<int64_t>(o_routed->size(0), 1) : 0;
  check(mb_decode_advance(reinterpret_cast<const long long*>(o_tok.data_ptr<int64_t>()), o_lp.data_ptr<float>(),
                          rec ? o_routed->data_ptr<int>() : nullptr, reinterpret_cast<long long*>(h_tok.data_ptr<int64_t>()),
                          h_lp.data_ptr<float>(), rec ? h_routed->data_ptr<int>() : nullptr, per, tok.data_ptr<int>(), pos.data_ptr<int>(),
                          len.data_ptr<int>(), block_table.data_ptr<int>(), block_table.size(1), block_size,
                          reinterpret_cast<long long*>(slot.data_ptr<int64_t>()), reinterpret_cast<long long*>(seed.data_ptr<int64_t>()), B,
                          static_cast<int>(vocab), error_flag.data_ptr<int>(), cur_stream()),
        "mb_decode_advance");
}

std::vector<at::Tensor> sample_logprob(const at::Tensor& logits, const at::Tensor& temperature, const at::Tensor& greedy,
                                       const c10::optional<at::Tensor>& seeds, int64_t step) {
  c10::cuda::CUDAGuard g(logits.device());
  const int64_t B = logits.size(0), V = logits.size(1);
  auto tok = at::empty({B}, logits.options().dtype(at::kLong));
  auto lp = at::empty({B}, logits.options());
  const long long* seed_ptr =
      seeds.has_value() && seeds->defined() ? reinterpret_cast<const long long*>(seeds->data_ptr<int64_t>()) : nullptr;
  // few rows: several CTAs per row (one CTA per row would leave a 150k-entry vocabulary to a single SM)
  const int64_t parts = std::min<int64_t>(32, 296 / std::max<int64_t>(B, 1));
  if (parts >= 2 && B <= 4096) {
    static std::vector<at::Tensor> counters(64);
    auto& cnt = counters[logits.device().index()];
    if (!cnt.defined()) cnt = at::zeros({4096}, logits.options().dtype(at::kInt));
    auto ws = at::empty({B * parts * 4}, logits.options());
    check(mb_sample_logprob_split(logits.data_ptr<float>(), temperature.data_ptr<float>(), greedy.data_ptr<uint8_t>(), seed_ptr, step,
                                  reinterpret_cast<long long*>(tok.data_ptr<int64_t>()), lp.data_ptr<float>(), B, V, parts,
                                  ws.data_ptr<float>(), cnt.data_ptr<int>(), cur_stream()),
          "mb_sample_logprob_split");
    return {tok, lp};
  }
  check(mb_sample_logprob(logits.data_ptr<float>(), temperature.data_ptr<float>(), greedy.data_ptr<uint8_t>(),
                          seeds.has_value() && seeds->defined() ? reinterpret_cast<const long long*>(seeds->data_ptr<int64_t>()) : nullptr,
                          step, reinterpret_cast<long long*>(tok.data_ptr<int64_t>()), lp.data_ptr<float>(), B, V, cur_stream()),
        "mb_sample_logprob");
  return {tok, lp};
}

void logit_stats(const at::Tensor& logits, const at::Tensor& targets, at::Tensor& stats, int64_t v0, double inv_temp, bool first) {
  c10::cuda::CUDAGuard g(logits.device());
  check(mb_logit_stats(logits.data_ptr<float>(), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                       stats.data_ptr<float>(), logits.size(0), logits.size(1), v0, inv_temp, first, cur_stream()),
        "mb_logit_stats");
}

void logit_stats_finish(const at::Tensor& stats, at::Tensor& logp, const c10::optional<at::Tensor>& ent,
                        const c10::optional<at::Tensor>& lse) {
  c10::cuda::CUDAGuard g(stats.device());
  check(mb_logit_stats_finish(stats.data_ptr<float>(), logp.data_ptr<float>(), fptr(ent), fptr(lse), stats.size(0), cur_stream()),
        "mb_logit_stats_finish");
}

void logit_grad(const at::Tensor& logits, const at::Tensor& targets, const at::Tensor& lse, const c10::optional<at::Tensor>& ent,
                const c10::optional<at::Tensor>& g_lp, const c10::optional<at::Tensor>& g_ent, at::Tensor& dlogits, int64_t v0,
                double inv_temp) {
  c10::cuda::CUDAGuard g(logits.device());
  check(mb_logit_grad(logits.data_ptr<float>(), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                      lse.data_ptr<float>(), fptr(ent), fptr(g_lp), fptr(g_ent), dlogits.data_ptr(), dlogits.stride(0), logits.size(0),
                      logits.size(1), v0, inv_temp, cur_stream()),
        "mb_logit_grad");
}

std::vector<at::Tensor> mxfp8_quant(const at::Tensor& x) {
  c10::cuda::CUDAGuard g(x.device());
  auto q = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
  auto sizes = x.sizes().vec();
  sizes.back() /= 32;
  auto sc = at::empty(sizes, x.options().dtype(at::kByte));
  check(mb_mxfp8_quant(x.data_ptr(), q.data_ptr(), sc.data_ptr(), x.numel(), cur_stream()), "mb_mxfp8_quant");
  return {q, sc};
}

std::vector<at::Tensor> fp8_block_quant(const at::Tensor& w) {
  c10::cuda::CUDAGuard g(w.device());
  const int64_t M = w.size(0), N = w.size(1);
  auto q = at::empty({M, N}, w.options().dtype(at::kFloat8_e4m3fn));
  auto sc = at::empty({(M + 127) / 128, (N + 127) / 128}, w.options().dtype(at::kFloat));
  check(mb_fp8_block_quant(w.data_ptr(), q.data_ptr(), sc.data_ptr<float>(), M, N, cur_stream()), "mb_fp8_block_quant");
  return {q, sc};
}

at::Tensor block_fake_quant(const at::Tensor& x, int64_t mode) {
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "block_fake_quant: contiguous bf16 input");
  at::Tensor y = at::empty_like(x);
  check(mb_block_fake_quant(x.data_ptr(), y.data_ptr(), x.numel(), static_cast<int>(mode), cur_stream()), "mb_block_fake_quant");
  return y;
}

std::vector<at::Tensor> int4_fake_quant(const at::Tensor& x, int64_t bm, int64_t bn, bool symmetric) {
  c10::cuda::CUDAGuard g(x.device());
  const int64_t M = x.size(0), N = x.size(1);
  auto y = at::empty_like(x);
  auto sc = at::empty({M / bm, N / bn}, x.options().dtype(at::kFloat));
  check(mb_int4_fake_quant(x.data_ptr(), y.data_ptr(), sc.data_ptr<float>(), M, N, bm, bn, symmetric, cur_stream()),
        "mb_int4_fake_quant");
  return {y, sc};
}

at::Tensor absmax(const at::Tensor& x) {
  c10::cuda::CUDAGuard g(x.device());
  auto out = at::zeros({1}, x.options().dtype(at::kFloat));
  check(mb_absmax(x.data_ptr(), out.data_ptr<float>(), x.numel(), cur_stream()), "mb_absmax");
  return out;
}

at::Tensor nvfp4_qdq(const at::Tensor& x, const at::Tensor& global_amax, bool four_over_six) {
  c10::cuda::CUDAGuard g(x.device());
  auto y = at::empty_like(x);
  check(mb_nvfp4_qdq(x.data_ptr(), y.data_ptr(), global_amax.data_ptr<float>(), x.numel(), four_over_six ? 1 : 0, cur_stream()), "mb_nvfp4_qdq");
  return y;
}

}  // namespace

void register_misc(pybind11::module& m) {
  m.def("decode_advance", &decode_advance);
  m.def("sample_logprob", &sample_logprob);
  m.def("logit_stats", &logit_stats);
  m.def("logit_stats_finish", &logit_stats_finish);
  m.def("logit_grad", &logit_grad);
  m.def("mxfp8_quant", &mxfp8_quant);
  m.def("fp8_block_quant", &fp8_block_quant);
  m.def("int4_fake_quant", &int4_fake_quant);
  m.def("block_fake_quant", &block_fake_quant);
  m.def("absmax", &absmax);
  m.def("nvfp4_qdq", &nvfp4_qdq);
  // index checks of the debug build: limits are published per kind of index (0 cache slots, 1 MoE (token, choice) pairs,
  // 2 cache blocks); the report lists, per translation unit, {count, first code, first index, its limit}
  m.def("is_debug_build", []() { return mb_elementwise_bounds_set_limit(-1, 0) != -1; });
  m.def("bounds_set_limit", [](int64_t which, int64_t value) {
    const int a = mb_elementwise_bounds_set_limit(which, value), b = mb_moe_bounds_set_limit(which, value),
              c = mb_paged_bounds_set_limit(which, value);
    return a == 0 && b == 0 && c == 0;
  });
  m.def("bounds_report", [](bool clear) {
    std::vector<std::vector<int64_t>> out;
    long long r[4];
    if (mb_elementwise_bounds_read(r, clear) == 0) out.push_back({0, r[0], r[1], r[2], r[3]});
    if (mb_moe_bounds_read(r, clear) == 0) out.push_back({1, r[0], r[1], r[2], r[3]});
    if (mb_paged_bounds_read(r, clear) == 0) out.push_back({2, r[0], r[1], r[2], r[3]});
    return out;
  });
}
