"""Tensor-parallel + sequence-parallel building blocks with autograd.

    column_parallel_linear : y = all_gather_seq(x) · Wᵀ          (W sharded by output rows)
    row_parallel_linear    : y = reduce_scatter_seq(x · Wᵀ)      (W sharded by input columns)
    vocab_parallel_logprob : log-softmax over a vocab-sharded LM head with max / sum all-reduces

Each has three executions chosen per call:
* CUDA + fabric + `ps.fused`: ONE sm_100a kernel per op that overlaps the NVLink transfer with the
  tcgen05 tiles (`fused_ag_gemm`, `fused_gemm_rs`, `fused_vocab_logprob` in the extension);
* CUDA without fabric (or `--disable-fused-comm`): NCCL collective + separate GEMM — the baseline the
  fused path is measured against, and what the reference does through Megatron's
  Column/RowParallelLinear (+ `fused_vocab_parallel_cross_entropy`,
  miles/backends/training_utils/loss/hub/math_utils.py:297-310, 423-459);
* CPU (gloo): the same collectives through `torch.distributed`, used by the multi-process tests.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops


# ---- raw collectives (no autograd) -------------------------------------------------------------

def _all_gather_dim0(x: torch.Tensor, ps) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty((x.shape[0] * ps.tp_size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x, group=ps.tp_group)
    else:
        dist.all_gather(list(out.chunk(ps.tp_size, 0)), x, group=ps.tp_group)
    return out


def _reduce_scatter_dim0(x: torch.Tensor, ps) -> torch.Tensor:
    x = x.contiguous()
    n = x.shape[0] // ps.tp_size
    if x.is_cuda:
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=ps.tp_group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=ps.tp_group)
    return y[ps.tp_rank * n:(ps.tp_rank + 1) * n].clone()


def _all_reduce(x: torch.Tensor, ps, op=dist.ReduceOp.SUM) -> torch.Tensor:
    y = x.contiguous().clone()
    dist.all_reduce(y, op=op, group=ps.tp_group)
    return y


def _use_fused(x: torch.Tensor, ps) -> bool:
    return x.is_cuda and ps.fabric is not None and ps.fused


# ---- sequence gather / scatter -----------------------------------------------------------------

class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ps):
        ctx.ps = ps
        return _all_gather_dim0(x, ps)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim0(g, ctx.ps), None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ps):
        ctx.ps = ps
        n = x.shape[0] // ps.tp_size
        return x[ps.tp_rank * n:(ps.tp_rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim0(g, ctx.ps), None


def gather_sequence(x, ps):
    return _GatherSeq.apply(x, ps)


def scatter_sequence(x, ps):
    return _ScatterSeq.apply(x, ps)


class _AllGatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ps):
        ctx.ps = ps
        parts = [torch.empty_like(x) for _ in range(ps.tp_size)]
        dist.all_gather(parts, x.contiguous(), group=ps.tp_group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        ps = ctx.ps
        return g.chunk(ps.tp_size, dim=-1)[ps.tp_rank].contiguous(), None


def all_gather_last_dim(x, ps):
    return _AllGatherLast.apply(x, ps)


# ---- column / row parallel linear -----------------------------------------------------------------

class _ColumnLinear(torch.autograd.Function):
    """x [T/tp, K] (sequence-parallel) or [T, K]; w [N/tp, K] → y [T, N/tp]."""

    @staticmethod
    def forward(ctx, x, w, bias, ps):
        ctx.ps = ps
        ctx.sp = ps.sequence_parallel
        if ctx.sp:
            if _use_fused(x, ps):
                y, xg = ps.fabric.ag_gemm(x, w, ps)          # fused all-gather → GEMM; also returns gathered x
            else:
                xg = _all_gather_dim0(x, ps)
                y = ops.linear(xg, w)
        else:
            xg = x
            y = ops.linear(x, w)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(xg if not ctx.sp else x, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        ps = ctx.ps
        gy = gy.contiguous()
        if ctx.sp:
            xg = _all_gather_dim0(x, ps)                     # re-gather instead of keeping [T,K] alive
            gx_full = ops.linear_dgrad(gy, w)
            if _use_fused(gy, ps):
                gx = ps.fabric.reduce_scatter(gx_full, ps)
            else:
                gx = _reduce_scatter_dim0(gx_full, ps)
        else:
            xg = x
            gx_full = ops.linear_dgrad(gy, w)
            gx = _all_reduce(gx_full, ps)
        gw = ops.linear_wgrad(gy, xg)
        gb = gy.sum(0) if ctx.has_bias else None
        return gx, gw, gb, None


class _RowLinear(torch.autograd.Function):
    """x [T, K/tp]; w [N, K/tp] → y [T/tp, N] (sequence-parallel) or [T, N] (all-reduced)."""

    @staticmethod
    def forward(ctx, x, w, ps):
        ctx.ps = ps
        ctx.sp = ps.sequence_parallel
        ctx.save_for_backward(x, w)
        if ctx.sp:
            if _use_fused(x, ps):
                return ps.fabric.gemm_rs(x, w, ps)          # fused GEMM → reduce-scatter
            return _reduce_scatter_dim0(ops.linear(x, w), ps)
        return _all_reduce(ops.linear(x, w), ps)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        ps = ctx.ps
        gy = gy.contiguous()
        if ctx.sp:
            if _use_fused(gy, ps):
                gx, gyg = ps.fabric.ag_gemm_dgrad(gy, w, ps)  # all-gather(gy) → gy·W fused
            else:
                gyg = _all_gather_dim0(gy, ps)
                gx = ops.linear_dgrad(gyg, w)
        else:
            gyg = gy
            gx = ops.linear_dgrad(gy, w)
        gw = ops.linear_wgrad(gyg, x)
        return gx, gw, None


def column_parallel_linear(x, w, bias, ps):
    return _ColumnLinear.apply(x, w, bias, ps)


def row_parallel_linear(x, w, ps):
    return _RowLinear.apply(x, w, ps)


# ---- vocab-parallel log-prob / entropy -------------------------------------------------------------

class _VocabParallelLogProb(torch.autograd.Function):
    """hidden [T,H] (replicated over TP), w [V/tp, H] → log p(target) [T], entropy [T].

    Forward: local logits chunk → all-reduce(MAX) of row maxima → all-reduce(SUM) of
    [Σexp, target logit, Σexp·logit].  Backward: d logits = g_lp·(onehot − p) + g_ent·(−p·(logit − E[logit]))
    formed per vocab shard, then dH all-reduced over TP.
    """

    @staticmethod
    def forward(ctx, hidden, w, targets, temperature, with_entropy, ps):
        Vl = w.shape[0]
        lo = ps.tp_rank * Vl
        logits = ops.linear(hidden, w).float()
        if temperature != 1.0:
            logits = logits / temperature
        mx = _all_reduce(logits.max(-1).values, ps, dist.ReduceOp.MAX)
        ex = torch.exp(logits - mx[:, None])
        local_t = targets.long() - lo
        inside = (local_t >= 0) & (local_t < Vl)
        tl = torch.where(inside, logits.gather(1, local_t.clamp(0, Vl - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
        pack = torch.stack([ex.sum(-1), tl, (ex * logits).sum(-1)], 0)
        pack = _all_reduce(pack, ps)
        sumexp, tlogit, sexl = pack[0], pack[1], pack[2]
        lse = mx + torch.log(sumexp)
        logp = tlogit - lse
        ent = lse - sexl / sumexp
        ctx.save_for_backward(hidden, w, targets, lse, ent)
        ctx.ps, ctx.temperature, ctx.with_entropy = ps, temperature, with_entropy
        return logp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, w, targets, lse, ent = ctx.saved_tensors
        ps, temp = ctx.ps, ctx.temperature
        Vl = w.shape[0]
        lo = ps.tp_rank * Vl
        logits = ops.linear(hidden, w).float()
        if temp != 1.0:
            logits = logits / temp
        p = torch.exp(logits - lse[:, None])
        local_t = targets.long() - lo
        inside = (local_t >= 0) & (local_t < Vl)
        dl = -p * g_lp[:, None]
        rows = torch.arange(p.shape[0], device=p.device)[inside]
        dl[rows, local_t[inside]] += g_lp[inside]
        if ctx.with_entropy and g_ent is not None:
            # dH/dlogit_j = −p_j (logit_j − Σ p·logit) = −p_j (logit_j − (lse − H))
            dl = dl - g_ent[:, None] * p * (logits - (lse - ent)[:, None])
        if temp != 1.0:
            dl = dl / temp
        dl = dl.to(hidden.dtype)
        gh = _all_reduce(dl @ w, ps)
        gw = dl.t() @ hidden
        return gh, gw, None, None, None, None


def vocab_parallel_logprob(hidden, w, targets, temperature, with_entropy, ps):
    if _use_fused(hidden, ps):
        return ps.fabric.vocab_logprob(hidden, w, targets, temperature, with_entropy, ps)
    logp, ent = _VocabParallelLogProb.apply(hidden, w, targets, temperature, with_entropy, ps)
    return logp, (ent if with_entropy else None)
