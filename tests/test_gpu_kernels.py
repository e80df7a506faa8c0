"""Numerics of the sm_100a kernels against plain-PyTorch fp32 statements of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from miles_b200.ops import reference as ref  # noqa: E402


def _k():
    from miles_b200.ops import cuda

    return cuda


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _flag_ok():
    assert _k().check_error_flag() == 0, "a kernel raised the bounded-wait error flag"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 1536, 2048), (4096, 4096, 1024), (64, 5120, 2048),
                                   (1, 2048, 2048), (300, 152, 1024)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_nt(M, N, K, bn):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = _k().gemm_nt(a, b, force_bn=bn)
    want = a.float() @ b.float().t()
    torch.cuda.synchronize()
    _flag_ok()
    assert _rel(out, want) < 1e-2, _rel(out, want)


@pytest.mark.parametrize("M,N,K", [(256, 512, 512), (1000, 2048, 1536), (4096, 1024, 4096)])
def test_gemm_nn_and_tn(M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    out = _k().gemm_nn(a, b)
    assert _rel(out, a.float() @ b.float()) < 1e-2
    at = torch.randn(K, M if M % 8 == 0 else M + 8 - M % 8, device="cuda", dtype=torch.bfloat16)
    out2 = _k().gemm_tn(at, b)
    assert _rel(out2, at.float().t() @ b.float()) < 1e-2
    acc = torch.ones(at.shape[1], N, device="cuda", dtype=torch.float32)
    _k().gemm_tn(at, b, out=acc, accumulate=True)
    assert _rel(acc, at.float().t() @ b.float() + 1.0) < 1e-2
    _flag_ok()


def test_gemm_bias_and_fp32_out():
    a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(768, device="cuda", dtype=torch.bfloat16)
    out = _k().gemm_nt(a, b, bias=bias, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    assert _rel(out, a.float() @ b.float().t() + bias.float()) < 5e-3


def test_linear_autograd():
    torch.manual_seed(2)
    x = torch.randn(777, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(1536, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = _k().linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(g.float())
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("T,H", [(1, 1024), (513, 2048), (300, 2560), (64, 5120), (70, 1024), (65, 4096), (63, 2048)])
def test_rmsnorm_fwd_bwd(T, H):
    torch.manual_seed(3)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y, rn = _k().add_rmsnorm(x, r, w, 1e-6)
    gy, gr = torch.randn_like(y), torch.randn_like(rn)
    torch.autograd.backward([y, rn], [gy, gr])
    xf, rf, wf = (t.detach().float().requires_grad_() for t in (x, r, w))
    s = xf + rf
    yr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    torch.autograd.backward([yr, s], [gy.float(), gr.float()])
    assert _rel(y, yr) < 1e-2 and _rel(rn, s) < 1e-2
    assert _rel(x.grad, xf.grad) < 2e-2 and _rel(r.grad, rf.grad) < 2e-2 and _rel(w.grad, wf.grad) < 2e-2
    y2 = _k().rmsnorm(x.detach(), w.detach(), 1e-6)
    assert _rel(y2, ref.rmsnorm(x.detach().float(), w.detach().float())) < 1e-2


def test_swiglu_fwd_bwd():
    x = torch.randn(1000, 2 * 768, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = _k().swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float().requires_grad_()
    a, b = xf.chunk(2, -1)
    (torch.nn.functional.silu(a) * b).backward(g.float())
    assert _rel(y, torch.nn.functional.silu(a) * b) < 1e-2 and _rel(x.grad, xf.grad) < 1e-2


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("norm", [True, False])
def test_qk_norm_rope(D, norm):
    torch.manual_seed(4)
    T, Hq, Hk = 333, 8, 2
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_() if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_() if norm else None
    pos = torch.randint(0, 30000, (T,), device="cuda", dtype=torch.int32)
    q, k, _ = qkv.split([Hq * D, Hk * D, Hk * D], dim=-1)
    qo, ko = _k().qk_norm_rope(q.view(T, Hq, D), k.view(T, Hk, D), qw, kw, pos, 1e6, 1e-6)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    torch.autograd.backward([qo, ko], [gq, gk])

    xf = qkv.detach().float().requires_grad_()
    qf, kf, _ = xf.split([Hq * D, Hk * D, Hk * D], dim=-1)
    qf, kf = qf.view(T, Hq, D), kf.view(T, Hk, D)
    if norm:
        qwf, kwf = qw.detach().float().requires_grad_(), kw.detach().float().requires_grad_()
        qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + 1e-6) * qwf
        kf = kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + 1e-6) * kwf
    qr, kr = ref.rope(qf, pos, 1e6), ref.rope(kf, pos, 1e6)
    torch.autograd.backward([qr, kr], [gq.float(), gk.float()])
    assert _rel(qo, qr) < 1e-2 and _rel(ko, kr) < 1e-2
    assert _rel(qkv.grad, xf.grad) < 2e-2
    if norm:
        assert _rel(qw.grad, qwf.grad) < 3e-2 and _rel(kw.grad, kwf.grad) < 3e-2


def test_adamw_matches_reference():
    n = 10007
    master = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    mask = (torch.rand(n, device="cuda") > 0.5).float()
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    mr, m_r, v_r = master.clone(), m.clone(), v.clone()
    for step in (1, 2, 3):
        _k().adamw_step_masked(master, g, m, v, mask, 1e-3, 0.9, 0.98, 1e-8, 0.1, step, 0.5, out)
        gs = g * 0.5
        m_r.mul_(0.9).add_(gs, alpha=0.1)
        v_r.mul_(0.98).addcmul_(gs, gs, value=0.02)
        denom = (v_r / (1 - 0.98 ** step)).sqrt() + 1e-8
        mr.mul_(1 - 1e-3 * 0.1 * mask).addcdiv_(m_r / (1 - 0.9 ** step), denom, value=-1e-3)
    assert torch.allclose(master, mr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(out.float(), mr, rtol=1e-2, atol=1e-2)


def test_kv_cache_write():
    T, H, D, bs = 50, 2, 128, 16
    k = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(8, bs, H, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(8 * bs, device="cuda")[:T]
    _k().kv_cache_write(k, v, kc, vc, slots)
    assert torch.equal(kc.view(-1, H, D)[slots], k) and torch.equal(vc.view(-1, H, D)[slots], v)


@pytest.mark.parametrize("M,N,K", [(1, 2048, 4096), (64, 2048, 4096), (64, 128, 2048), (8, 4096, 2048), (200, 1000, 3072), (130, 152, 1024)])
@pytest.mark.parametrize("fp32_out", [False, True])
def test_gemm_split_k(M, N, K, fp32_out, monkeypatch):
    """Decode-sized GEMMs go through the split-K path; results match, and the arrival counters are left zero."""
    K_ = _k()
    monkeypatch.setattr(K_, "_SPLITK_MAX_M", 256)           # the dispatch default only splits very small M
    assert K_._pick_split_k(M, N, K) > 1
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    want = a.float() @ b.float().t() + bias.float()
    for _ in range(3):                                       # back to back: each call must find a clean workspace
        out = K_.gemm_nt(a, b, bias=bias, out_dtype=torch.float32 if fp32_out else None)
        torch.cuda.synchronize()
        _flag_ok()
        assert _rel(out, want) < (2e-3 if fp32_out else 1e-2), _rel(out, want)
    nob = K_.gemm_nt(a, b, out_dtype=torch.float32 if fp32_out else None)          # vectorised reduction path
    assert _rel(nob, want - bias.float()) < (2e-3 if fp32_out else 1e-2)
    ws, counters = K_._splitk_workspace(a.device)
    assert int(counters.abs().max()) == 0
    plain = K_.gemm_nt(a, b, bias=bias, out_dtype=torch.float32, force_bn=64)     # force_bn bypasses split-K
    assert _rel(out.float(), plain) < 1e-2


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("norm", [True, False])
def test_qk_norm_rope_cache_matches_separate_ops(D, norm):
    K_ = _k()
    torch.manual_seed(2)
    T, Hq, Hk, bs, nb = 37, 8, 2, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv.split([Hq * D, Hk * D, Hk * D], dim=-1)
    q, k, v = q.view(T, Hq, D), k.view(T, Hk, D), v.view(T, Hk, D)
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16() if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16() if norm else None
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(bs * nb, device="cuda")[:T].to(torch.int64)
    slots[5] = -1                                             # a token that is not cached
    kc0 = torch.randn(nb, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    vc0 = torch.randn(nb, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        q1, k1 = K_.qk_norm_rope(q, k, qw, kw, pos, 1e6, 1e-6)
        kc1, vc1 = kc0.clone(), vc0.clone()
        K_.kv_cache_write(k1, v, kc1, vc1, slots)
        kc2, vc2 = kc0.clone(), vc0.clone()
        q2, k2 = K_.qk_norm_rope_cache(q, k, v, qw, kw, pos, 1e6, 1e-6, kc2, vc2, slots)
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(k1, k2)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)


@pytest.mark.parametrize("D,H,T", [(128, 8, 300), (64, 3, 17)])
def test_rope_alone_and_swiglu_fp32(D, H, T):
    """The stand-alone rotary kernel (forward, inverse, autograd) and the fp32-compute SwiGLU against their fp32 statements."""
    from miles_b200.ops import extra

    torch.manual_seed(4)
    x = torch.randn(T, H, D, device="cuda").to(torch.bfloat16).requires_grad_()
    pos = torch.randint(0, 40000, (T,), device="cuda", dtype=torch.int32)
    y = _k().rope(x, pos, 1e6)
    want = ref.rope(x.detach().float(), pos, 1e6)
    assert _rel(y, want) < 1e-2
    back = _k().rope(y.detach(), pos, 1e6, inverse=True)
    assert _rel(back, x.detach().float()) < 2e-2                       # inverse rotation returns the input
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float().requires_grad_()
    ref.rope(xf, pos, 1e6).backward(g.float())
    assert _rel(x.grad, xf.grad) < 1e-2
    strided = torch.randn(T, H * D + 64, device="cuda").to(torch.bfloat16)[:, : H * D].view(T, H, D)     # token stride ≠ H·D
    assert _rel(_k().rope(strided, pos, 1e4), ref.rope(strided.float(), pos, 1e4)) < 1e-2
    gu = torch.randn(T, 2 * 384, device="cuda").to(torch.bfloat16)
    a, b = gu.float().chunk(2, -1)
    assert _rel(extra.swiglu_fp32(gu), torch.nn.functional.silu(a) * b) < 1e-2
