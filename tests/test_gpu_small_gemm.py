"""Numerics of the decode-sized GEMMs (weights on the 128-row MMA side, tokens in tiles of 16/32/64) vs fp32 PyTorch."""
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


@pytest.mark.parametrize("M", [1, 7, 16, 17, 32, 50, 64])
@pytest.mark.parametrize("N,K", [(128, 2048), (5120, 2048), (2048, 4096), (200, 328), (1536, 256)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_small_matches_fp32(M, N, K, out_dtype):
    torch.manual_seed(M + N)
    K_ = _k()
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    assert M <= K_.SMALL_M
    y = K_.gemm_nt(x, w, bias=bias, out_dtype=out_dtype)
    y2 = K_.gemm_nt(x, w, bias=bias, out_dtype=out_dtype)              # the split-K counters must be back at zero
    expect = x.float() @ w.float().t() + bias.float()
    assert y.dtype == out_dtype and _rel(y, expect) < (5e-3 if out_dtype == torch.bfloat16 else 1e-4)
    assert torch.equal(y, y2)
    assert K_.check_error_flag(x) == 0


def test_gemm_small_every_split_and_tile():
    K_ = _k()
    torch.manual_seed(0)
    x = torch.randn(40, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(384, 1024, device="cuda", dtype=torch.bfloat16) * 0.05
    expect = x.float() @ w.float().t()
    ws = torch.empty(16 * 40 * 384, dtype=torch.float32, device="cuda")
    counters = torch.zeros(4 * 64, dtype=torch.int32, device="cuda")
    for bt in (16, 32, 64):
        for split in (1, 2, 4, 16):
            out = torch.empty(40, 384, dtype=torch.float32, device="cuda")
            K_.C.gemm_small(x, w, out, 40, 384, 1024, 384, None, bt, split, ws, counters)
            assert _rel(out, expect) < 1e-4, (bt, split)
            assert int(counters.abs().sum()) == 0
    assert K_.check_error_flag(x) == 0


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(128, 2048), (5120, 2048), (2048, 4096), (1000, 96)])
def test_gemv_matches_fp32(M, N, K):
    K_ = _k()
    torch.manual_seed(M * 7 + N)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    expect = x.float() @ w.float().t() + bias.float()
    for static_w in (False, True):
        y = torch.empty(M, N, device="cuda", dtype=torch.float32)
        K_.C.gemv(x, None, None, 0.0, w, bias, y, None, None, static_w)
        assert _rel(y, expect) < 1e-4
    yb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    K_.C.gemv(x, None, None, 0.0, w, None, yb, None, None, False)
    assert _rel(yb, expect - bias.float()) < 5e-3


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rmsnorm_linear_matches_unfused(M, with_residual):
    K_ = _k()
    torch.manual_seed(M)
    K, N, eps = 2048, 640, 1e-6
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) if with_residual else None
    nw = (1 + 0.1 * torch.randn(K, device="cuda")).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    old = K_.GEMV_M
    K_.GEMV_M = 16
    try:
        with torch.no_grad():
            assert K_.gemv_ok(x, w)
            y, res, xn = K_.add_rmsnorm_linear(x, r, nw, eps, w, want_normed=True)
    finally:
        K_.GEMV_M = old
    h = (x.float() + r.float()).to(torch.bfloat16).float() if with_residual else x.float()
    xn_ref = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * nw.float()
    assert _rel(xn, xn_ref) < 5e-3
    assert _rel(y, xn_ref @ w.float().t()) < 1e-2
    if with_residual:
        assert torch.equal(res.float(), h)
    else:
        assert res is None


def test_gemm_small_strided_output():
    K_ = _k()
    x = torch.randn(5, 512, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16) * 0.05
    buf = torch.zeros(5, 1024, device="cuda", dtype=torch.bfloat16)
    K_.gemm_nt(x, w, out=buf[:, 256:512])
    assert _rel(buf[:, 256:512], x.float() @ w.float().t()) < 5e-3
    assert float(buf[:, :256].abs().sum()) == 0 and float(buf[:, 512:].abs().sum()) == 0


@pytest.mark.parametrize("T,E,K,H,F", [(1, 8, 2, 256, 128), (9, 16, 4, 512, 256), (64, 128, 8, 2048, 768), (200, 16, 2, 256, 128)])
def test_moe_ffn_small_tiles_match_fp32(T, E, K, H, F):
    from miles_b200.ops import cuda_more

    torch.manual_seed(T)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13 = torch.randn(E, 2 * F, H, device="cuda", dtype=torch.bfloat16) * 0.03
    w2 = torch.randn(E, H, F, device="cuda", dtype=torch.bfloat16) * 0.03
    logits = torch.randn(T, E, device="cuda")
    tw, ti = logits.softmax(-1).topk(K, dim=-1)
    expect = ref.moe_ffn(x.float(), w13.float(), w2.float(), tw, ti)
    with torch.no_grad():
        bt = cuda_more.small_moe_bt(T * K, E, w13, w2)
        assert bt in (16, 32, 64)
        y = cuda_more.moe_ffn(x, w13, w2, tw, ti)
        for forced in (16, 32, 64):
            y_f = cuda_more._moe_ffn_small(x, w13, w2, tw, ti, 0, forced)
            assert _rel(y_f, expect) < 2e-2, forced
    assert _rel(y, expect) < 2e-2
    y_train = cuda_more.moe_ffn(x.requires_grad_(), w13, w2, tw, ti)        # autograd on: the 128-row path
    assert _rel(y, y_train) < 1e-2
    assert _k().check_error_flag(x) == 0


@pytest.mark.parametrize("T,E,K,H,F", [(1, 128, 8, 2048, 768), (8, 128, 8, 2048, 768), (5, 4, 4, 256, 96), (3, 16, 2, 128, 32)])
def test_moe_gemv_matches_fp32(T, E, K, H, F):
    from miles_b200.ops import cuda_more

    torch.manual_seed(T + E)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13 = torch.randn(E, 2 * F, H, device="cuda", dtype=torch.bfloat16) * 0.03
    w2 = torch.randn(E, H, F, device="cuda", dtype=torch.bfloat16) * 0.03
    tw, ti = torch.randn(T, E, device="cuda").softmax(-1).topk(K, dim=-1)
    expect = ref.moe_ffn(x.float(), w13.float(), w2.float(), tw, ti)
    n0 = _k().launch_count()
    with torch.no_grad():
        y = cuda_more.moe_ffn(x, w13, w2, tw, ti)
    assert _k().launch_count() - n0 == 2                     # the two matrix-vector kernels, nothing else
    assert _rel(y, expect) < 2e-2
    # experts split over two "ranks": the halves add up
    with torch.no_grad():
        lo = cuda_more.moe_ffn(x, w13[: E // 2], w2[: E // 2], tw, ti, 0)
        hi = cuda_more.moe_ffn(x, w13[E // 2:], w2[E // 2:], tw, ti, E // 2)
    assert _rel(lo.float() + hi.float(), expect) < 2e-2


def test_moe_ffn_small_expert_offset():
    from miles_b200.ops import cuda_more

    torch.manual_seed(3)
    T, E, K, H, F = 12, 8, 2, 256, 128
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13 = torch.randn(E, 2 * F, H, device="cuda", dtype=torch.bfloat16) * 0.03
    w2 = torch.randn(E, H, F, device="cuda", dtype=torch.bfloat16) * 0.03
    tw, ti = torch.randn(T, E, device="cuda").softmax(-1).topk(K, dim=-1)
    with torch.no_grad():
        full = cuda_more.moe_ffn(x, w13, w2, tw, ti)
        lo = cuda_more.moe_ffn(x, w13[:4], w2[:4], tw, ti, 0)
        hi = cuda_more.moe_ffn(x, w13[4:], w2[4:], tw, ti, 4)
    assert _rel(lo.float() + hi.float(), full) < 1e-2
