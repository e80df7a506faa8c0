"""Ops of the other model families (hyper-connections, short convolutions, per-layer embeddings, grouped norms) and of the
quantisation tools.  Reference kernels: miles/kernels/norm/grouped_rmsnorm.py:13-78, activation/swiglu_fp32.py:8-124,
activation/short_conv_fp32.py:9-144, hyper_connection/hc.py:16-246, hyper_connection/mhc.py:6-185,
embedding/ple_gather.py:12-64, quant/fp8_act_quant.py:47-137, tools/fp8_cast_bf16.py:16.

Every op has a plain-PyTorch fp32 statement (`*_ref`: the CPU path and the test oracle, differentiable) and, on CUDA,
a one-pass sm_100a forward kernel (`ops/csrc/extra.cu`); backward passes apply the analytic gradients with tensor ops.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _C():
    from . import cuda

    return cuda.C


# ---- grouped RMSNorm -------------------------------------------------------------------------------------------

def grouped_rmsnorm_ref(x, w, n: int, eps: float):
    T, W = x.shape
    C = W // n
    xf = x.float().view(T, n, C)
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * (1.0 + w.float().view(n, C))).view(T, W), rstd.view(T, n)


class _GroupedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, n, eps):
        x = x.contiguous()
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        rstd = torch.empty(x.shape[0], n, dtype=torch.float32, device=x.device)
        _C().grouped_rmsnorm(x, w.float().contiguous(), out, rstd, n, eps)
        ctx.save_for_backward(x, w, rstd)
        ctx.n = n
        return out

    @staticmethod
    def backward(ctx, g):
        x, w, rstd = ctx.saved_tensors
        n = ctx.n
        T, W = x.shape
        C = W // n
        xh = x.float().view(T, n, C) * rstd.view(T, n, 1)
        gw = g.float().view(T, n, C) * (1.0 + w.float().view(n, C))
        dx = rstd.view(T, n, 1) * (gw - xh * (gw * xh).mean(-1, keepdim=True))
        dw = (g.float().view(T, n, C) * xh).sum(0).view_as(w)
        return dx.view(T, W).to(x.dtype), dw.to(w.dtype), None, None


def grouped_rmsnorm(x, w, n: int, eps: float = 1e-6):
    """x [T, n·C] → fp32 [T, n·C]: RMS norm of each of the n streams of a token, scaled by (1 + w)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
        return _GroupedRMSNorm.apply(x, w, n, eps)
    return grouped_rmsnorm_ref(x, w, n, eps)[0]


# ---- SwiGLU in fp32 ------------------------------------------------------------------------------------------------

def swiglu_fp32(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate)·up computed in fp32, rounded once to the input dtype (matches the engine's `silu_and_mul`)."""
    if gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and gate_up.shape[-1] % 16 == 0:
        # the SwiGLU kernel reads bf16, computes silu(gate)·up in fp32 registers and rounds once: exactly this contract
        from .. import ops

        return ops.swiglu(gate_up.reshape(-1, gate_up.shape[-1])).reshape(*gate_up.shape[:-1], gate_up.shape[-1] // 2)
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


# ---- short causal depthwise convolution over packed sequences --------------------------------------------------------

def _bos(seqlens, T: int, device) -> torch.Tensor:
    """Index of the first token of each token's sequence."""
    if seqlens is None:
        return torch.zeros(T, dtype=torch.int32, device=device)
    lens = torch.as_tensor(seqlens, device=device, dtype=torch.long)
    starts = torch.cumsum(lens, 0) - lens
    return torch.repeat_interleave(starts, lens).to(torch.int32)


def short_conv_ref(x, weight, seqlens=None):
    T, D = x.shape
    W = weight.shape[1]
    bos = _bos(seqlens, T, x.device).long()
    t = torch.arange(T, device=x.device)
    acc = x.float().clone()
    for iw in range(W):
        s = t - (W - 1) + iw
        ok = (s >= bos).unsqueeze(1)
        acc = acc + torch.where(ok, x.float()[s.clamp_min(0)], torch.zeros((), device=x.device)) * weight.float()[:, iw]
    return acc.to(x.dtype)


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bos):
        x = x.contiguous()
        y = torch.empty_like(x)
        _C().short_conv(x, weight.float().contiguous(), bos, y)
        ctx.save_for_backward(x, weight, bos)
        return y

    @staticmethod
    def backward(ctx, g):
        x, weight, bos = ctx.saved_tensors
        T, D = x.shape
        W = weight.shape[1]
        t = torch.arange(T, device=x.device)
        gf, xf = g.float(), x.float()
        dx = gf.clone()
        dw = torch.zeros(D, W, dtype=torch.float32, device=x.device)
        b = bos.long()
        for iw in range(W):
            shift = (W - 1) - iw                         # y[t] reads x[t − shift] when t − shift ≥ bos[t]
            src = t - shift
            ok = (src >= b)
            contrib = gf * weight.float()[:, iw] * ok.unsqueeze(1)
            dx.index_add_(0, src.clamp_min(0), contrib)
            dw[:, iw] = (gf * xf[src.clamp_min(0)] * ok.unsqueeze(1)).sum(0)
        return dx.to(x.dtype), dw.to(weight.dtype), None


def short_conv_fp32(x, weight, seqlens=None):
    """y[t] = x[t] + Σ_i w[:, i]·x[t − (W−1) + i] within each packed sequence (fp32 accumulation)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
        return _ShortConv.apply(x, weight, _bos(seqlens, x.shape[0], x.device))
    return short_conv_ref(x, weight, seqlens)


# ---- hyper-connections ---------------------------------------------------------------------------------------------

def mhc_mix_ref(x, residual, h_res, h_post, n: int):
    lead, d = x.shape[:-1], x.shape[-1]
    r = residual.float().reshape(*lead, n, d)
    out = h_post.float().unsqueeze(-1) * x.float().unsqueeze(-2) + torch.einsum("...ij,...id->...jd", h_res.float(), r)
    return out.reshape(*lead, n * d).to(x.dtype)


def mhc_mix(x, residual, h_res, h_post, n: int):
    """out_j = h_post_j · x + Σ_i h_res[i, j] · residual_i, flattened to [..., n·d]."""
    if x.is_cuda and not torch.is_grad_enabled() and x.dtype in (torch.bfloat16, torch.float32):
        lead, d = x.shape[:-1], x.shape[-1]
        x2, r2 = x.reshape(-1, d).contiguous(), residual.reshape(-1, n * d).contiguous()
        out = torch.empty_like(r2)
        _C().mhc_mix(x2, r2, h_res.float().reshape(-1, n * n).contiguous(), h_post.float().reshape(-1, n).contiguous(), out, n)
        return out.reshape(*lead, n * d)
    return mhc_mix_ref(x, residual, h_res, h_post, n)


def mhc_aggregate_ref(x, pre, n: int):
    lead = x.shape[:-1]
    d = x.shape[-1] // n
    return (pre.float().unsqueeze(-1) * x.float().reshape(*lead, n, d)).sum(-2)


def mhc_aggregate(x, pre, n: int):
    """Σ_i pre_i · x_i in fp32 without the [..., n, d] temporary."""
    if x.is_cuda and not torch.is_grad_enabled() and x.dtype in (torch.bfloat16, torch.float32):
        lead = x.shape[:-1]
        d = x.shape[-1] // n
        x2 = x.reshape(-1, n * d).contiguous()
        out = torch.empty(x2.shape[0], d, dtype=torch.float32, device=x.device)
        _C().mhc_aggregate(x2, pre.float().reshape(-1, n).contiguous(), out, n)
        return out.reshape(*lead, d)
    return mhc_aggregate_ref(x, pre, n)


def hc_combine_ref(residual, block_output, h_post, n: int):
    lead = residual.shape[:-1]
    C = block_output.shape[-1]
    out = residual.float().reshape(*lead, n, C) + h_post.float().reshape(*lead, n, 1) * block_output.float().unsqueeze(-2)
    return out.reshape(*lead, n * C).to(residual.dtype)


def hc_combine(residual, block_output, h_post, n: int):
    """X'_c = X_c + a_c · y for the n residual streams."""
    if residual.is_cuda and not torch.is_grad_enabled() and residual.dtype in (torch.bfloat16, torch.float32):
        lead, C = residual.shape[:-1], block_output.shape[-1]
        r2, y2 = residual.reshape(-1, n * C).contiguous(), block_output.reshape(-1, C).contiguous()
        out = torch.empty_like(r2)
        _C().hc_combine(r2, y2.to(r2.dtype), h_post.float().reshape(-1, n).contiguous(), out, n)
        return out.reshape(*lead, n * C)
    return hc_combine_ref(residual, block_output, h_post, n)


def hc_mix_inject(x, weight, w_down, w_up, w_inject, n: int, eps: float):
    """Grouped norm → gate chain → gated mean over the streams (`mixed` [T, C]) and the injection gate (`h_post` [T, n]):
        normed = grouped_rmsnorm(x);  gate = σ(W_up · silu(W_down · normed / n));  mixed = mean_i(gate_i ⊙ normed_i)
        h_post = 2 σ(W_inject · normed / n)"""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    T, W = x2.shape
    C = W // n
    normed = grouped_rmsnorm(x2, weight, n, eps)
    gate = torch.sigmoid(F.linear(F.silu(F.linear(normed, w_down.float()) / n), w_up.float()))
    mixed = (gate * normed).view(T, n, C).mean(1).to(x.dtype).reshape(*lead, C)
    h_post = None
    if w_inject is not None:
        h_post = (2.0 * torch.sigmoid(F.linear(normed, w_inject.float()) / n)).reshape(*lead, n)
    return mixed, h_post


# ---- per-layer embeddings: rows from a pinned host table ----------------------------------------------------------------

def gather_rows_host(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """`table` [rows, width] in pinned host memory, `ids` int64 on the device → [..., width] on the device.  The kernel
    reads the host rows through the mapped address (no staging copy, no host synchronisation)."""
    flat = ids.reshape(-1).to(torch.int64)
    if ids.is_cuda and table.is_pinned() and (table.shape[1] * table.element_size()) % 16 == 0:
        out = torch.empty(flat.numel(), table.shape[1], dtype=table.dtype, device=ids.device)
        _C().gather_rows_host(table, flat.contiguous(), out)
    else:
        out = table[flat.cpu().clamp(0, table.shape[0] - 1)].to(ids.device)
        out[(flat < 0) | (flat >= table.shape[0])] = 0
    return out.reshape(*ids.shape, table.shape[1])


# ---- FP8 activation quantisation (1×128) and block dequantisation -------------------------------------------------------

def act_quant_ref(x, block: int = 128, round_scale: bool = False):
    M, N = x.shape
    xb = x.float().view(M, N // block, block)
    amax = xb.abs().amax(-1).clamp_min(1e-4)
    s = amax / 448.0
    if round_scale:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (xb / s.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(M, N), s


def act_quant(x, block: int = 128, round_scale: bool = False, inplace: bool = False):
    """Per-row 1×128 FP8 e4m3 quantisation.  Returns (q, scales) — or, with `inplace`, (x quantised-and-dequantised in
    bf16, scales), the fake-quant used for quantisation-aware training."""
    assert block == 128 and x.dim() == 2 and x.shape[1] % 128 == 0
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x.contiguous()
        scales = torch.empty(x.shape[0], x.shape[1] // 128, dtype=torch.float32, device=x.device)
        if inplace:
            out = torch.empty_like(x)
            _C().act_quant_1x128(x, None, out, scales, round_scale)
            return out, scales
        q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        _C().act_quant_1x128(x, q, None, scales, round_scale)
        return q.view(torch.float8_e4m3fn), scales
    q, s = act_quant_ref(x, block, round_scale)
    if inplace:
        return (q.float().view(x.shape[0], -1, block) * s.unsqueeze(-1)).view_as(x).to(x.dtype), s
    return q, s


def gemm_mxfp8_ref(a_q, a_s, b_q, b_s) -> torch.Tensor:
    """fp32 statement of the block-scaled product: dequantise both operands, multiply."""
    from . import reference as ref

    a = ref.mxfp8_dequant(a_q, a_s).reshape(a_q.shape).float()
    b = ref.mxfp8_dequant(b_q, b_s).reshape(b_q.shape).float()
    return a @ b.t()


def gemm_mxfp8(a_q, a_s, b_q, b_s, out: torch.Tensor | None = None) -> torch.Tensor:
    """C [M, N] bf16 = MXFP8(A) · MXFP8(B)ᵀ with A [M, K], B [N, K] e4m3 and e8m0 scales [rows, K/32] (what `mxfp8_quant`
    returns).  On CUDA the scales are applied inside the tensor core (tcgen05 block-scaled MMA); K % 128 == 0."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if a_q.is_cuda and K % 128 == 0:
        from . import cuda

        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=a_q.device)
        cuda.C.gemm_mxfp8(a_q.contiguous().view(torch.uint8), a_s.contiguous(), b_q.contiguous().view(torch.uint8), b_s.contiguous(), out,
                          cuda.C.error_flag(out))
        return out
    res = gemm_mxfp8_ref(a_q, a_s, b_q, b_s).bfloat16()
    if out is not None:
        out.copy_(res)
        return out
    return res


def gemm_mxfp8_grouped(a_q, a_s, b_q, b_s, tile_expert, out: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped (MoE) block-scaled product.  a_q [M_pad, K] e4m3 with scales [M_pad, K/32]: expert-sorted rows whose segments are
    padded to 128; b_q [E, N, K] with scales [E, N, K/32]; `tile_expert` int32 [M_pad/128] names the expert of every row block
    (−1: block not in use, left untouched).  C [M_pad, N] bf16; N % 128 == 0, K % 128 == 0."""
    M, K = a_q.shape
    E, N, _ = b_q.shape
    if a_q.is_cuda and K % 128 == 0 and N % 128 == 0 and M % 128 == 0:
        from . import cuda

        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=a_q.device)
        cuda.C.gemm_mxfp8_grouped(a_q.contiguous().view(torch.uint8), a_s.contiguous(), b_q.contiguous().view(torch.uint8), b_s.contiguous(),
                                  out, tile_expert, cuda.C.error_flag(out))
        return out
    from . import reference as ref

    res = torch.zeros(M, N, dtype=torch.float32, device=a_q.device) if out is None else out.float()
    a = ref.mxfp8_dequant(a_q, a_s).reshape(M, K).float()
    for blk, e in enumerate(tile_expert.tolist()):
        if e >= 0:
            b = ref.mxfp8_dequant(b_q[e], b_s[e]).reshape(N, K).float()
            res[blk * 128:(blk + 1) * 128] = a[blk * 128:(blk + 1) * 128] @ b.t()
    res = res.bfloat16()
    if out is not None:
        out.copy_(res)
        return out
    return res


def linear_mxfp8(x: torch.Tensor, w_q: torch.Tensor, w_s: torch.Tensor) -> torch.Tensor:
    """y = x·Wᵀ with W held in MXFP8 (weights quantised once, e.g. by the weight sync) and x quantised on the fly."""
    from .. import ops

    xq, xs = ops.mxfp8_quant(x.reshape(-1, x.shape[-1]))
    return gemm_mxfp8(xq, xs, w_q, w_s).view(*x.shape[:-1], w_q.shape[0])


def fp8_dequant(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Block-scaled FP8 weight → bf16.  `scale` fp32 [⌈M/128⌉, ⌈N/128⌉] (scale_inv of 128×128 blocks) or uint8 e8m0
    [M, N/32] (MXFP8)."""
    from . import reference as ref

    M, N = q.shape
    if q.is_cuda and N % 4 == 0:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=q.device)
        q8 = q.contiguous().view(torch.uint8)
        if scale.dtype == torch.uint8:
            _C().fp8_dequant(q8, None, scale.contiguous(), out)
        else:
            _C().fp8_dequant(q8, scale.float().contiguous(), None, out)
        return out
    if scale.dtype == torch.uint8:
        return ref.mxfp8_dequant(q, scale).reshape(M, N).bfloat16()
    return ref.fp8_blockwise_dequant(q, scale)
