

def test_block_fake_quant_reference_grids_scales_and_straight_through():
    """MXFP8 / MXFP4 / compressed-KV style fake quantisation: values land on (payload grid × block scale), scales are powers
    of two (e4m3 numbers for the compressed-KV style), the block maximum is representable, and the gradient passes through."""
    import torch

    from miles_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(8, 128) * torch.logspace(-3, 2, 8)[:, None]
    grid4 = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6.0])
    for mode, block in (("fp8", 32), ("fp4", 32), ("compressed_kv", 16)):
        xin = x.clone().requires_grad_(True)
        y = ops.block_fake_quant(xin, mode)
        y.sum().backward()
        assert torch.equal(xin.grad, torch.ones_like(x))                      # straight-through
        yb, xb = y.detach().reshape(-1, block), x.reshape(-1, block)
        amax = xb.abs().amax(1)
        fmax = 448.0 if mode == "fp8" else 6.0
        if mode == "compressed_kv":
            scale = (amax / 6).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn).float()
        else:
            scale = torch.exp2(torch.ceil(torch.log2(amax.clamp_min(1e-4 if mode == "fp8" else 1e-37) / fmax)))
        q = (yb / scale[:, None]).abs()
        if mode == "fp8":
            assert torch.equal(q.to(torch.float8_e4m3fn).float(), q) and float(q.max()) <= 448
            assert float(((yb - xb).abs() / xb.abs().clamp_min(1e-6))[xb.abs() > amax[:, None] / 16].max()) < 0.07
        else:
            assert bool(((q[..., None] - grid4).abs().amin(-1) < 1e-6).all())
            assert float((yb - xb).abs().max() / amax.max()) <= 0.26
    b = torch.tensor([[6.0, 0.25, 0.75, 1.75, 2.5, 3.5, 5.0, -5.0] + [0.0] * 24])
    assert ops.block_fake_quant(b, "fp4")[0, :8].tolist() == [6.0, 0.0, 1.0, 2.0, 2.0, 4.0, 4.0, -4.0]   # ties to even
