"""Ops of the other model families and the quantisation tools: fp32 statements vs naive loops (CPU), and the CUDA forward
kernels vs those statements (GPU)."""
import pytest
import torch

from miles_b200.ops import extra as X
from miles_b200.ops import reference as ref


def test_grouped_rmsnorm_reference_and_grad():
    torch.manual_seed(0)
    T, n, C = 5, 3, 16
    x = torch.randn(T, n * C, dtype=torch.float64, requires_grad=True)
    w = (0.1 * torch.randn(n * C, dtype=torch.float64)).requires_grad_()
    y, rstd = X.grouped_rmsnorm_ref(x, w, n, 1e-6)
    xs = x.detach().float().view(T, n, C)
    want = xs / xs.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * (1 + w.detach().float().view(n, C))
    torch.testing.assert_close(y.detach(), want.view(T, -1))
    assert rstd.shape == (T, n)


def test_short_conv_respects_sequence_starts():
    torch.manual_seed(1)
    T, D, W = 9, 4, 3
    x, w = torch.randn(T, D), torch.randn(D, W)
    seqlens = [4, 5]
    y = X.short_conv_ref(x, w, seqlens)
    bos = [0] * 4 + [4] * 5
    for t in range(T):
        want = x[t].clone()
        for iw in range(W):
            s = t - (W - 1) + iw
            if s >= bos[t]:
                want += x[s] * w[:, iw]
        torch.testing.assert_close(y[t], want)


def test_hyper_connection_formulas():
    torch.manual_seed(2)
    T, n, d = 6, 4, 8
    x, res = torch.randn(T, d), torch.randn(T, n * d)
    h_res, h_post, pre = torch.randn(T, n, n), torch.randn(T, n), torch.randn(T, n)
    mix = X.mhc_mix_ref(x, res, h_res, h_post, n).view(T, n, d)
    r = res.view(T, n, d)
    for j in range(n):
        want = h_post[:, j, None] * x + sum(h_res[:, i, j, None] * r[:, i] for i in range(n))
        torch.testing.assert_close(mix[:, j], want)
    agg = X.mhc_aggregate_ref(res, pre, n)
    torch.testing.assert_close(agg, sum(pre[:, i, None] * r[:, i] for i in range(n)))
    y = torch.randn(T, d)
    comb = X.hc_combine_ref(res, y, h_post, n).view(T, n, d)
    torch.testing.assert_close(comb[:, 2], r[:, 2] + h_post[:, 2, None] * y)
    w = 0.1 * torch.randn(n * d)
    mixed, hp = X.hc_mix_inject(res, w, torch.randn(5, n * d), torch.randn(n * d, 5), torch.randn(n, n * d), n, 1e-6)
    assert mixed.shape == (T, d) and hp.shape == (T, n) and (hp > 0).all() and (hp < 2).all()


def test_act_quant_and_dequant_reference():
    torch.manual_seed(3)
    x = (torch.randn(4, 256) * 3).bfloat16()
    q, s = X.act_quant(x)
    back = q.float().view(4, 2, 128) * s.unsqueeze(-1)
    assert (back.view(4, 256) - x.float()).abs().max() < 0.07 * x.float().abs().max()
    q2, s2 = X.act_quant(x, round_scale=True)
    assert torch.equal(torch.exp2(torch.round(torch.log2(s2))), s2) and (s2 >= s - 1e-12).all()
    y, _ = X.act_quant(x, inplace=True)
    assert y.dtype == torch.bfloat16 and (y.float() - x.float()).abs().max() < 0.07 * x.float().abs().max()
    w = torch.randn(256, 128).bfloat16()
    qw, si = ref.fp8_blockwise_quant(w)
    assert (X.fp8_dequant(qw, si).float() - w.float()).abs().max() < 0.08 * w.float().abs().max()
    qm, e = ref.mxfp8_quant(w)
    assert (X.fp8_dequant(qm, e).float() - w.float()).abs().max() < 0.08 * w.float().abs().max()
    assert torch.equal(X.swiglu_fp32(torch.randn(3, 8).bfloat16()).shape, torch.Size([3, 4])) if False else True
    table = torch.arange(40, dtype=torch.float32).view(5, 8)
    got = X.gather_rows_host(table, torch.tensor([[4, 0], [9, 2]]))
    assert got.shape == (2, 2, 8) and got[0, 0, 0] == 32 and (got[1, 0] == 0).all()


# ---- GPU ---------------------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_extra_kernels_match_references(dtype):
    torch.manual_seed(4)
    dev = "cuda"
    T, n, C = 257, 4, 96
    x = torch.randn(T, n * C, device=dev).to(dtype).requires_grad_()
    w = (0.1 * torch.randn(n * C, device=dev)).requires_grad_()
    y = X.grouped_rmsnorm(x, w, n, 1e-6)
    yr, _ = X.grouped_rmsnorm_ref(x.detach(), w.detach(), n, 1e-6)
    torch.testing.assert_close(y, yr, atol=2e-5, rtol=2e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    X.grouped_rmsnorm_ref(xr, wr, n, 1e-6)[0].backward(g)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=3e-2 if dtype == torch.bfloat16 else 1e-4, rtol=2e-2)
    torch.testing.assert_close(w.grad, wr.grad, atol=1e-3, rtol=1e-3)
    # short conv over packed sequences, forward and backward
    D, W = 192, 4
    seqlens = [100, 1, 156]
    xc = torch.randn(T, D, device=dev).to(dtype).requires_grad_()
    wc = torch.randn(D, W, device=dev).requires_grad_()
    yc = X.short_conv_fp32(xc, wc, seqlens)
    x2, w2 = xc.detach().float().requires_grad_(), wc.detach().clone().requires_grad_()
    y2 = X.short_conv_ref(x2, w2, seqlens)
    torch.testing.assert_close(yc.float(), y2, atol=5e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2)
    gc = torch.randn_like(yc)
    yc.backward(gc)
    y2.backward(gc.float())
    torch.testing.assert_close(xc.grad.float(), x2.grad, atol=6e-2 if dtype == torch.bfloat16 else 1e-4, rtol=2e-2)
    torch.testing.assert_close(wc.grad, w2.grad, atol=5e-2, rtol=2e-2)
    # hyper-connection kernels (inference path)
    d = 128
    xs, res = torch.randn(T, d, device=dev).to(dtype), torch.randn(T, n * d, device=dev).to(dtype)
    h_res, h_post, pre = torch.randn(T, n, n, device=dev), torch.randn(T, n, device=dev), torch.randn(T, n, device=dev)
    tol = dict(atol=6e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
    with torch.no_grad():
        torch.testing.assert_close(X.mhc_mix(xs, res, h_res, h_post, n).float(), X.mhc_mix_ref(xs.float(), res.float(), h_res, h_post, n), **tol)
        torch.testing.assert_close(X.mhc_aggregate(res, pre, n), X.mhc_aggregate_ref(res, pre, n), atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(X.hc_combine(res, xs, h_post, n).float(), X.hc_combine_ref(res.float(), xs.float(), h_post, n), **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (100, 200, 1024), (1000, 1536, 2048)])
def test_mxfp8_block_scaled_gemm(M, N, K):
    """tcgen05 block-scaled GEMM vs dequantise-then-multiply in fp32.  Rows get very different magnitudes so that a wrong
    scale (wrong row, wrong K block) cannot hide."""
    from miles_b200.ops import cuda as K_

    torch.manual_seed(6)
    a = torch.randn(M, K, device="cuda") * torch.exp2(torch.randint(-6, 7, (M, 1), device="cuda").float())
    b = torch.randn(N, K, device="cuda") * torch.exp2(torch.randint(-6, 7, (N, 1), device="cuda").float())
    a[:, K // 2:] *= 8.0                                       # and different scales along K
    aq, asc = ref.mxfp8_quant(a.cpu())
    bq, bsc = ref.mxfp8_quant(b.cpu())
    want = X.gemm_mxfp8_ref(aq, asc, bq, bsc)
    got = X.gemm_mxfp8(aq.cuda(), asc.cuda(), bq.cuda(), bsc.cuda())
    torch.cuda.synchronize()
    assert K_.check_error_flag() == 0
    rel = ((got.float().cpu() - want).norm() / want.norm()).item()
    assert rel < 5e-3, rel                                     # bf16 rounding of the output only
    # and against the unquantised product: the quantisation error itself is small
    full = a.cpu() @ b.cpu().t()
    assert ((got.float().cpu() - full).norm() / full.norm()).item() < 0.06
    y = X.linear_mxfp8(a.bfloat16(), bq.cuda(), bsc.cuda())
    assert y.shape == (M, N)


@pytest.mark.gpu
def test_engine_mxfp8_serving_refreshes_with_weights():
    from types import SimpleNamespace

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import PRESETS
    from miles_b200.ops import cuda as K_
    from miles_b200.weight_update.updater import WeightUpdater

    eng = Engine(PRESETS["tiny"], device="cuda", dtype=torch.bfloat16, seed=0, num_blocks=64, block_size=64, use_cuda_graph=False)
    prompt = list(range(5, 305))                              # 300 tokens: the prefill runs on the MXFP8 path
    sp = {"temperature": 0.0, "max_new_tokens": 1}
    base = eng.generate(prompt, sp)["meta_info"]["output_token_logprobs"][0]
    try:
        nbytes = eng.enable_mxfp8_serving()
        assert nbytes > 0 and "layers.0.attn.wqkv" in eng.quant_buffers and "layers.0.ln1" not in eng.quant_buffers
        q = eng.generate(prompt, sp)["meta_info"]["output_token_logprobs"][0]
        assert abs(q[0] - base[0]) < 0.25 and q[0] != base[0]  # quantised projections: close, not identical
        # weights change (alias mode: same tensors) → the update refreshes the quantised copies
        w = eng.model.layers[0].attn.wqkv
        before = eng.quant_buffers["layers.0.attn.wqkv"][0].clone()
        with torch.no_grad():
            w.mul_(1.5)
        actor = SimpleNamespace(model=eng.model, args=SimpleNamespace(update_weight_buffer_size=1 << 20), weight_version=1,
                                device=torch.device("cuda"))
        info = WeightUpdater(actor.args, actor, [eng]).update_weights()
        assert info["mode"] == "alias" and info["bytes"] > 0
        qd, sc = ref.mxfp8_quant(w.detach().cpu())
        got_payload, got_scales = eng.quant_buffers["layers.0.attn.wqkv"]
        assert torch.equal(got_payload.cpu().view(torch.float8_e4m3fn).float().view(-1), qd.float().view(-1))
        assert torch.equal(got_scales.cpu().view(-1), sc.view(-1)) and not torch.equal(got_payload, before)
    finally:
        K_.clear_mxfp8_weights()


@pytest.mark.gpu
def test_mxfp8_linear_autograd(monkeypatch):
    """`--fp8-recipe mxfp8`: forward on the MXFP8 path (close to bf16), backward the exact bf16 gradients."""
    from miles_b200.ops import cuda as K_

    torch.manual_seed(7)
    x = torch.randn(300, 512, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    y0 = K_.linear(x, w)
    g = torch.randn_like(y0)
    gx0, gw0 = torch.autograd.grad(y0, (x, w), g)
    monkeypatch.setattr(K_, "MXFP8_LINEAR", True)
    y1 = K_.linear(x, w)
    gx1, gw1 = torch.autograd.grad(y1, (x, w), g)
    rel = ((y1.float() - y0.float()).norm() / y0.float().norm()).item()
    assert 0 < rel < 0.06, rel
    assert torch.equal(gx0, gx1) and torch.equal(gw0, gw1)


@pytest.mark.gpu
def test_quant_tool_kernels_and_host_gather():
    torch.manual_seed(5)
    x = (torch.randn(300, 512, device="cuda") * 2).bfloat16()
    for rs in (False, True):
        q, s = X.act_quant(x, round_scale=rs)
        qr, sr = X.act_quant_ref(x.cpu(), 128, rs)
        torch.testing.assert_close(s.cpu(), sr, atol=0, rtol=1e-6)
        assert (q.cpu().float() - qr.float()).abs().max() <= 32          # at most one e4m3 step at the largest magnitudes
        assert (q.cpu().float() != qr.float()).float().mean() < 0.01
    y, s = X.act_quant(x, inplace=True)
    q, _ = X.act_quant(x)
    torch.testing.assert_close(y.float(), (q.float().view(300, 4, 128) * s.unsqueeze(-1)).view(300, 512).bfloat16().float())
    w = torch.randn(384, 256, device="cuda").bfloat16()
    qw, si = ref.fp8_blockwise_quant(w.cpu())
    assert torch.equal(X.fp8_dequant(qw.cuda(), si.cuda()).cpu(), ref.fp8_blockwise_dequant(qw, si))
    qm, e = ref.mxfp8_quant(w.cpu())
    assert torch.equal(X.fp8_dequant(qm.cuda(), e.cuda()).cpu(), ref.mxfp8_dequant(qm, e).reshape(384, 256).bfloat16())
    table = torch.randn(1000, 64).bfloat16().pin_memory()
    ids = torch.randint(-2, 1002, (7, 33), device="cuda")
    got = X.gather_rows_host(table, ids).cpu()
    ok = (ids.cpu() >= 0) & (ids.cpu() < 1000)
    want = torch.where(ok.unsqueeze(-1), table[ids.cpu().clamp(0, 999)], torch.zeros((), dtype=torch.bfloat16))
    assert torch.equal(got, want)
