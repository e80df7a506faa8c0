"""Numerics of the attention / MoE / log-prob / sampling / quantisation kernels vs fp32 PyTorch statements."""
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


def _attn_ref(q, k, v, cu, causal=True):
    return ref.attention_varlen(q.float(), k.float(), v.float(), cu, causal)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("lens", [[1], [64], [65, 3, 200], [513, 128, 77, 1000]])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2)])
def test_flash_attention_fwd_bwd(D, lens, heads):
    torch.manual_seed(0)
    Hq, Hkv = heads
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    o = _k().attention_varlen(q.view(T, Hq, D), k.view(T, Hkv, D), v.view(T, Hkv, D), cu, max(lens))
    g = torch.randn_like(o)
    o.backward(g)
    xf = qkv.detach().float().requires_grad_()
    qf, kf, vf = xf.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    of = _attn_ref(qf.view(T, Hq, D), kf.view(T, Hkv, D), vf.view(T, Hkv, D), cu)
    of.backward(g.float())
    assert _rel(o, of) < 2e-2, _rel(o, of)
    assert _rel(qkv.grad, xf.grad) < 3e-2, _rel(qkv.grad, xf.grad)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens", [[1], [127], [128], [129], [4096], [300, 1, 129, 64, 1000]])
@pytest.mark.parametrize("heads", [(8, 1), (4, 4)])
def test_flash_attention_bwd_tcgen05_vs_fp32(lens, heads, causal):
    """The tcgen05 backward (head_dim 128) against fp32 autograd, and against the mma.sync backward it replaces."""
    from miles_b200.ops import cuda_more

    torch.manual_seed(1)
    Hq, Hkv = heads
    D, T = 128, sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    grads = {}
    for tc in (True, False):
        cuda_more.USE_TC_ATTENTION_BWD = tc
        try:
            qkv = (0.5 * torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
                   ).to(torch.bfloat16).requires_grad_()
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            o = cuda_more._FlashAttn.apply(q.view(T, Hq, D), k.view(T, Hkv, D), v.view(T, Hkv, D), cu, max(lens), causal)
            g = torch.randn(o.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(4)).to(torch.bfloat16)
            o.backward(g)
            grads[tc] = qkv.grad.clone()
        finally:
            cuda_more.USE_TC_ATTENTION_BWD = True
    assert _k().check_error_flag() == 0
    xf = qkv.detach().float().requires_grad_()
    qf, kf, vf = xf.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    of = _attn_ref(qf.view(T, Hq, D), kf.view(T, Hkv, D), vf.view(T, Hkv, D), cu, causal)
    of.backward(g.float())
    for name, lo, hi in (("dq", 0, Hq * D), ("dk", Hq * D, (Hq + Hkv) * D), ("dv", (Hq + Hkv) * D, (Hq + 2 * Hkv) * D)):
        want = xf.grad[:, lo:hi]
        if want.norm() < 1e-4:         # a single-key softmax has no gradient towards q and k: only rounding noise may remain
            assert grads[True][:, lo:hi].float().abs().max() < 1e-4, name
            continue
        assert _rel(grads[True][:, lo:hi], want) < 3e-2, (name, _rel(grads[True][:, lo:hi], want))
        assert _rel(grads[True][:, lo:hi], grads[False][:, lo:hi]) < 3e-2, (name, "vs mma.sync")


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 32, 4), (128, 8, 8), (64, 4, 2)])
def test_paged_decode(D, Hq, Hkv):
    torch.manual_seed(1)
    bs, nblocks, B = 64, 64, 5
    kc = torch.randn(nblocks, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nblocks, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    seq_lens = torch.tensor([1, 63, 64, 65, 700], dtype=torch.int32, device="cuda")
    perm = torch.randperm(nblocks)[: B * 11].view(B, 11).to(torch.int32).cuda()
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    out = _k().paged_attention(q, kc, vc, perm, seq_lens)
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), perm, seq_lens)
    assert _rel(out, want) < 2e-2, _rel(out, want)


def test_router_topk_matches_reference():
    torch.manual_seed(2)
    T, E, K = 1000, 128, 8
    logits = torch.randn(T, E, device="cuda", requires_grad=True)
    w, idx, probs = _k().router_topk(logits, K, True)
    lr = logits.detach().clone().requires_grad_()
    wr, ir, pr = ref.router_topk(lr, K, True)
    assert torch.equal(idx.long().sort(-1).values, ir.long().sort(-1).values)
    assert torch.allclose(probs, pr, atol=1e-6)
    assert torch.allclose(w.sort(-1).values, wr.sort(-1).values, atol=1e-6)
    g = torch.randn_like(w)
    # compare gradients with the same (sorted-by-index) slot order
    order, order_r = idx.long().argsort(-1), ir.long().argsort(-1)
    (w.gather(1, order) * g).sum().backward()
    (wr.gather(1, order_r) * g).sum().backward()
    assert torch.allclose(logits.grad, lr.grad, atol=1e-5)


@pytest.mark.parametrize("T,E,K,H,F", [(64, 8, 2, 256, 128), (1000, 16, 8, 1024, 384), (3, 16, 4, 512, 256)])
def test_moe_ffn_fwd_bwd(T, E, K, H, F):
    torch.manual_seed(3)
    x = (0.5 * torch.randn(T, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    w13 = (0.05 * torch.randn(E, 2 * F, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    w2 = (0.05 * torch.randn(E, H, F, device="cuda")).to(torch.bfloat16).requires_grad_()
    logits = torch.randn(T, E, device="cuda")
    tw, ti, _ = ref.router_topk(logits, K, True)
    tw = tw.detach().requires_grad_()
    y = _k().moe_ffn(x, w13, w2, tw, ti)
    g = torch.randn_like(y)
    y.backward(g)
    assert _k().check_error_flag() == 0
    xf, w13f, w2f, twf = (t.detach().float().requires_grad_() for t in (x, w13, w2, tw))
    yf = ref.moe_ffn(xf, w13f, w2f, twf, ti)
    yf.backward(g.float())
    assert _rel(y, yf) < 2e-2, _rel(y, yf)
    assert _rel(x.grad, xf.grad) < 3e-2, _rel(x.grad, xf.grad)
    assert _rel(w13.grad, w13f.grad) < 3e-2, _rel(w13.grad, w13f.grad)
    assert _rel(w2.grad, w2f.grad) < 3e-2, _rel(w2.grad, w2f.grad)
    assert _rel(tw.grad, twf.grad) < 3e-2, _rel(tw.grad, twf.grad)


def test_moe_ffn_expert_offset_skips_foreign_experts():
    torch.manual_seed(4)
    T, E, K, H, F = 200, 8, 2, 256, 128
    x = (0.5 * torch.randn(T, H, device="cuda")).to(torch.bfloat16)
    w13 = (0.05 * torch.randn(E, 2 * F, H, device="cuda")).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(E, H, F, device="cuda")).to(torch.bfloat16)
    tw, ti, _ = ref.router_topk(torch.randn(T, 2 * E, device="cuda"), K, True)   # ids in [0, 16); this rank owns [8, 16)
    y = _k().moe_ffn(x, w13, w2, tw, ti, expert_offset=E)
    mask = (ti >= E)
    want = ref.moe_ffn(x.float(), w13.float(), w2.float(), tw * mask, (ti - E).clamp_min(0))
    assert _rel(y, want) < 2e-2


@pytest.mark.parametrize("R,H,V,temp", [(100, 256, 1000, 1.0), (700, 1024, 40000, 0.7)])
def test_logprob_entropy_fwd_bwd(R, H, V, temp):
    torch.manual_seed(5)
    h = torch.randn(R, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (R,), device="cuda")
    lp, ent = _k().logprob_entropy(h, w, tg, temp, True)
    g1, g2 = torch.randn_like(lp), torch.randn_like(ent)
    torch.autograd.backward([lp, ent], [g1, g2])
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = (hf @ wf.t()) / temp
    lse = torch.logsumexp(logits, -1)
    lpr = logits.gather(1, tg[:, None]).squeeze(1) - lse
    entr = lse - (torch.softmax(logits, -1) * logits).sum(-1)
    torch.autograd.backward([lpr, entr], [g1, g2])
    assert torch.allclose(lp, lpr, atol=2e-2, rtol=1e-2), (lp - lpr).abs().max()
    assert torch.allclose(ent, entr, atol=2e-2, rtol=1e-2)
    assert _rel(h.grad, hf.grad) < 3e-2, _rel(h.grad, hf.grad)
    assert _rel(w.grad, wf.grad) < 3e-2, _rel(w.grad, wf.grad)


def test_sample_logprob_distribution_and_logprob():
    torch.manual_seed(6)
    V = 50
    logits = torch.randn(1, V, device="cuda").repeat(20000, 1)
    temp = torch.full((20000,), 0.8, device="cuda")
    greedy = torch.zeros(20000, dtype=torch.bool, device="cuda")
    seeds = torch.arange(20000, device="cuda")
    tok, lp = _k().sample_logprob(logits, temp, greedy, seeds, 3)
    p = torch.softmax(logits[0] / 0.8, -1)
    freq = torch.bincount(tok, minlength=V).float() / 20000
    assert (freq - p).abs().max() < 0.02
    assert torch.allclose(lp, torch.log(p)[tok], atol=1e-4)
    tok_g, lp_g = _k().sample_logprob(logits[:4], temp[:4], torch.ones(4, dtype=torch.bool, device="cuda"), None, 0)
    assert (tok_g == logits[0].argmax()).all()


def test_quant_kernels_match_reference():
    torch.manual_seed(7)
    x = (torch.randn(256, 512, device="cuda") * torch.rand(256, 1, device="cuda") * 10).to(torch.bfloat16)
    q, s = _k().mxfp8_quant(x)
    qr, sr = ref.mxfp8_quant(x)
    assert torch.equal(s, sr)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    w = torch.randn(300, 520, device="cuda").to(torch.bfloat16)
    q, si = _k().fp8_blockwise_quant(w)
    qr, sir = ref.fp8_blockwise_quant(w)
    assert torch.allclose(si, sir, rtol=1e-6)
    assert _rel(ref.fp8_blockwise_dequant(q, si, dtype=torch.float32), ref.fp8_blockwise_dequant(qr, sir, dtype=torch.float32)) < 1e-3
    for sym in (True, False):
        for bm, bn in ((1, 32), (32, 1), (16, 16)):
            y, sc = _k().int4_fake_quant(x, bm, bn, sym)
            yr, scr = ref.int4_fake_quant(x, bm, bn, sym)
            assert _rel(y, yr) < 2e-2, (sym, bm, bn, _rel(y, yr))
    y = _k().nvfp4_qdq(x)
    yr = ref.nvfp4_qdq(x)
    assert _rel(y, yr) < 2e-2, _rel(y, yr)
    assert (y != yr).float().mean() < 1e-3                       # same grid points except rare ties of the reciprocal
    # four-over-six: per block the better of "max → 6" and "max → 4"; never worse than the plain rule
    y46 = _k().nvfp4_qdq(x, None, True)
    yr46 = ref.nvfp4_qdq(x, four_over_six=True)
    assert (y46 != yr46).float().mean() < 1e-3
    e, e46 = (y.float() - x.float()).pow(2).sum(), (y46.float() - x.float()).pow(2).sum()
    assert e46 < e
    # the packed export decodes to the same values
    from miles_b200.weight_update import quant_export as qe

    x2 = x.reshape(-1, 64)
    assert (qe.nvfp4_dequantize(*qe.nvfp4_quantize(x2, four_over_six=True)) != y46.reshape(-1, 64)).float().mean() < 1e-3


def test_fused_weight_sync_kernels():
    """One launch per bucket: byte copy (odd sizes, unaligned tail) and MXFP8 quantise / quantise-dequantise on the way."""
    from types import SimpleNamespace

    from miles_b200.parallel.weight_sync import fused_weight_sync

    class M(torch.nn.Module):
        def __init__(self, seed):
            super().__init__()
            g = torch.Generator(device="cuda").manual_seed(seed)
            mk = lambda *s, dt=torch.bfloat16: torch.nn.Parameter(torch.randn(*s, device="cuda", generator=g).to(dt))
            self.ln1 = mk(257)                               # 514 bytes: not a multiple of 16
            self.wqkv = mk(384, 256)
            self.w2 = mk(3, 128, 96)                         # stacked experts
            self.head_bias = mk(1001, dt=torch.float32)
            self.w_small = mk(5, 7)

    src, dst = M(1), M(2)
    actor = SimpleNamespace(model=src, args=SimpleNamespace(update_weight_buffer_size=64 << 10))
    engine = SimpleNamespace(model=dst)
    n = fused_weight_sync(actor, engine)
    assert n == sum(p.numel() * p.element_size() for p in src.parameters())
    for (name, p), (_, q) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(p, q), name
    # quantise → dequantise on the way: 2-D+ weights whose rows are multiples of 32 change, the rest are copied
    dst2 = M(3)
    fused_weight_sync(actor, SimpleNamespace(model=dst2), quant="mxfp8_qdq")
    for name in ("wqkv", "w2"):
        p = getattr(src, name).detach()
        qd, sc = ref.mxfp8_quant(p)
        want = ref.mxfp8_dequant(qd, sc).reshape(p.shape).bfloat16()
        assert torch.equal(getattr(dst2, name).detach(), want), name
    assert torch.equal(dst2.ln1, src.ln1) and torch.equal(dst2.w_small, src.w_small)
    # payload + scales form
    eng3 = SimpleNamespace(model=M(4), quant_buffers={
        n_: (torch.empty(p.numel(), dtype=torch.uint8, device="cuda"), torch.empty(p.numel() // 32, dtype=torch.uint8, device="cuda"))
        for n_, p in src.named_parameters() if n_ in ("wqkv", "w2")})
    fused_weight_sync(actor, eng3, quant="mxfp8")
    for name in ("wqkv", "w2"):
        p = getattr(src, name).detach()
        qd, sc = ref.mxfp8_quant(p)
        payload, scales = eng3.quant_buffers[name]
        assert torch.equal(payload.view(torch.float8_e4m3fn).float().view(-1), qd.float().view(-1)), name
        assert torch.equal(scales.view(-1), sc.view(-1)), name


@pytest.mark.parametrize("heads", [(8, 1), (4, 4)])
@pytest.mark.parametrize("case", [[(1, 1)], [(5, 133)], [(128, 128)], [(64, 1000), (1, 65), (200, 200), (129, 4096)]])
def test_extend_attention_separate_query_and_key_sequences(case, heads):
    """New tokens attending to their request's paged KV (a cached prefix, an earlier piece of a chunked prompt): the tcgen05
    forward with separate query and key sequences against the fp32 statement over the paged cache."""
    torch.manual_seed(5)
    Hq, Hkv = heads
    D, bs = 128, 64
    q_lens = [c[0] for c in case]
    k_lens = [c[1] for c in case]
    B = len(case)
    nb = [(L + bs - 1) // bs for L in k_lens]
    total_blocks = sum(nb) + 3
    kc = torch.randn(total_blocks, bs, Hkv, D, device="cuda").mul_(0.5).to(torch.bfloat16)
    vc = torch.randn(total_blocks, bs, Hkv, D, device="cuda").mul_(0.5).to(torch.bfloat16)
    perm = torch.randperm(total_blocks)[: sum(nb)].tolist()                 # scattered blocks
    bt = torch.zeros(B, max(nb), dtype=torch.int32, device="cuda")
    at = 0
    for b in range(B):
        bt[b, : nb[b]] = torch.tensor(perm[at:at + nb[b]], dtype=torch.int32)
        at += nb[b]
    q = torch.randn(sum(q_lens), Hq, D, device="cuda").mul_(0.5).to(torch.bfloat16)
    sl = torch.tensor(k_lens, dtype=torch.int32, device="cuda")
    ql = torch.tensor(q_lens, dtype=torch.int32, device="cuda")
    got = _k().paged_attention(q, kc, vc, bt, sl, ql, max(q_lens))
    want = ref.paged_attention(q.float(), kc.float(), vc.float(), bt, sl, q_lens=ql)
    assert _k().check_error_flag() == 0
    assert _rel(got, want) < 2e-2, _rel(got, want)


def test_grouped_mxfp8_gemm_and_moe_forward():
    """The grouped (MoE) block-scaled GEMM against the fp32 product of the dequantised operands, with uneven expert
    segments, an unused expert and unused row blocks; then the MoE layer forward under the MXFP8 recipe against bf16."""
    from miles_b200.ops import cuda as K
    from miles_b200.ops import extra

    torch.manual_seed(7)
    E, N, Kd = 5, 256, 512
    rows = [300, 0, 128, 17, 260]                                  # tokens per expert
    pad = [(r + 127) // 128 * 128 for r in rows]
    M_pad = sum(pad) + 256                                         # two unused row blocks at the end
    tile_expert = torch.full((M_pad // 128,), -1, dtype=torch.int32)
    a = torch.zeros(M_pad, Kd)
    at = 0
    for e, (r, p) in enumerate(zip(rows, pad)):
        a[at:at + r] = torch.randn(r, Kd)
        tile_expert[at // 128:(at + p) // 128] = e
        at += p
    a = a.cuda().to(torch.bfloat16)
    b = (torch.randn(E, N, Kd) * 0.5).cuda().to(torch.bfloat16)
    tile_expert = tile_expert.cuda()
    aq, as_ = _k().mxfp8_quant(a)
    bq, bs = _k().mxfp8_quant(b.reshape(E * N, Kd))
    out = torch.full((M_pad, N), 7.0, dtype=torch.bfloat16, device="cuda")
    extra.gemm_mxfp8_grouped(aq, as_, bq.view(E, N, Kd), bs.view(E, N, Kd // 32), tile_expert, out=out)
    assert K.check_error_flag() == 0
    a_d = ref.mxfp8_dequant(aq.cpu(), as_.cpu()).reshape(M_pad, Kd).float()
    b_d = ref.mxfp8_dequant(bq.cpu(), bs.cpu()).reshape(E, N, Kd).float()
    at = 0
    for e, (r, p) in enumerate(zip(rows, pad)):
        if r:
            want = a_d[at:at + r] @ b_d[e].t()
            assert _rel(out[at:at + r].float().cpu(), want) < 1e-2, e
        at += p
    assert bool((out[at:] == 7.0).all())                           # unused row blocks are not written
    # the MoE layer under the recipe: forward close to bf16 (quantisation noise), backward identical (straight-through)
    T, H, F, k = 1400, 256, 128, 2
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_()
    w13 = (torch.randn(E, 2 * F, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(E, H, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).cuda().to(torch.int32)
    tw = torch.rand(T, k, device="cuda")
    outs = {}
    for flag in (False, True):
        K.MXFP8_LINEAR = flag
        try:
            y = _k().moe_ffn(x, w13, w2, tw, idx)
            y.float().pow(2).sum().backward()
            outs[flag] = (y.detach().float(), x.grad.clone(), w13.grad.clone())
            x.grad = w13.grad = w2.grad = None
        finally:
            K.MXFP8_LINEAR = False
    # e4m3 keeps 3 mantissa bits: two chained products of quantised operands land within ≈ 7 % of bf16
    assert 1e-3 < _rel(outs[True][0], outs[False][0]) < 0.1        # really quantised, and close
    assert _rel(outs[True][1], outs[False][1]) < 0.15 and _rel(outs[True][2], outs[False][2]) < 0.15


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp8", "fp4", "compressed_kv"])
def test_block_fake_quant_kernel_matches_the_reference_bit_for_bit(mode):
    """One-pass quantise → dequantise (1×32 power-of-two scales with e4m3 / e2m1 payloads, 1×16 e4m3 scales with e2m1)
    against the fp32 PyTorch statement of the same arithmetic, over magnitudes from 1e-4 to 1e3 and exact zeros."""
    from miles_b200 import ops
    from miles_b200.ops import reference as ref

    torch.manual_seed(3)
    x = (torch.randn(512, 4096, device="cuda") * torch.logspace(-4, 3, 512, device="cuda")[:, None]).bfloat16()
    x[7] = 0
    x[9, ::3] = 0
    want = ref.block_fake_quant(x, mode)
    xin = x.clone().requires_grad_(True)
    got = ops.block_fake_quant(xin, mode)
    assert got.dtype == torch.bfloat16 and torch.equal(got, want), float((got.float() - want.float()).abs().max())
    got.sum().backward()
    assert torch.equal(xin.grad, torch.ones_like(x))


@pytest.mark.gpu
def test_linear_mxfp8_backward_matches_fp32_gradients_within_block_scaling_error():
    """`--fp8-backward`: dgrad contracts over N and wgrad over the tokens, each on operands quantised 1×32 along that axis;
    against fp32 gradients the relative error stays at the e4m3 level (≈ 4–5 %), and the switch really changes the result."""
    from miles_b200.ops import cuda as K

    torch.manual_seed(5)
    M, N, Kd = 512, 768, 1024
    x = (torch.randn(M, Kd, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16().requires_grad_()
    gy = torch.randn(M, N, device="cuda").bfloat16()
    ref_gx = gy.float() @ w.detach().float()
    ref_gw = gy.float().t() @ x.detach().float()
    old = (K.MXFP8_LINEAR, K.MXFP8_BACKWARD)
    try:
        K.MXFP8_LINEAR = True
        grads = {}
        for flag in (False, True):
            K.MXFP8_BACKWARD = flag
            x.grad = w.grad = None
            K.linear(x, w).backward(gy)
            grads[flag] = (x.grad.float().clone(), w.grad.float().clone())
    finally:
        K.MXFP8_LINEAR, K.MXFP8_BACKWARD = old
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(grads[False][0], ref_gx) < 1e-2 and rel(grads[False][1], ref_gw) < 1e-2          # bf16 gradient GEMMs
    assert 1e-3 < rel(grads[True][0], ref_gx) < 7e-2 and 1e-3 < rel(grads[True][1], ref_gw) < 7e-2
    assert K.check_error_flag() == 0
