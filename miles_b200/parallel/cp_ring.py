"""Context-parallel attention without a head swap: ring (p2p, zigzag layout) and all-gather (contiguous layout).

The reference's default CP is Megatron/TE ring attention over a zigzag token layout (`cp_comm_type = ["p2p"]`,
miles/backends/megatron_utils/arguments.py:62-63; slicing in training_utils/data/context_parallel.py:250-297) and
`--allgather-cp` gathers K/V for contiguous chunks (data/rollout.py:233-269).  Both are written here against an explicit
description of which global tokens each rank holds, so any layout works:

* `token_index(total, ps)`: global positions (in the packed micro-batch) of the tokens this rank holds;
* `ring_attention`: K/V chunks travel around the CP group (cp − 1 exchanges), each rank folds the partial attention of
  its queries against the visiting chunk into a running (output, log-sum-exp) pair; the backward pass sends the chunk
  round again together with its gradient accumulators, which arrive home after the last step;
* `allgather_attention`: K/V are all-gathered (differentiably: the gradient is reduce-scattered) and every rank
  attends from its queries to the whole batch.

Visibility is decided per (query, key) from the sequence id and the position inside the sequence, so packed batches,
padding tokens (their own trailing pseudo-sequence) and both layouts need no special cases.  The block math is plain
PyTorch on both CPU and GPU (quadratic temporaries per chunk pair): this is the functional path; the long-context
production path on one NVSwitch box is the Ulysses layout (`cp.py`), which keeps the tcgen05 attention kernel.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from . import cp as _cp


def layout_mode(ps) -> str:
    if ps.cp_comm_type == "a2a+p2p":
        return "hier"
    return "zigzag" if ps.cp_comm_type == "p2p" else "contiguous"


def rank_token_index(total: int, cp_size: int, rank: int, mode: str, device=None) -> torch.Tensor:
    if mode == "zigzag":
        parts = [torch.arange(lo, hi, device=device) for lo, hi in _cp.zigzag_bounds(total, cp_size, rank)]
        return torch.cat(parts)
    lo, hi = _cp.chunk_bounds(total, cp_size, rank)
    return torch.arange(lo, hi, device=device)


def token_index(total: int, ps, device=None) -> torch.Tensor:
    """Global indices of the tokens of a length-`total` packed batch held by this CP rank (layout by `cp_comm_type`).
    Hierarchical (`a2a+p2p`): the ring member's two zigzag pieces, cut evenly over the members of its all-to-all group."""
    if layout_mode(ps) == "hier":
        a, i, o = ps.cp_a2a_size, ps.cp_rank % ps.cp_a2a_size, ps.cp_rank // ps.cp_a2a_size
        piece = rank_token_index(total, ps.cp_p2p_size, o, "zigzag", device)
        n = piece.numel() // a
        return piece[i * n:(i + 1) * n]
    return rank_token_index(total, ps.cp_size, ps.cp_rank, layout_mode(ps), device)


def _seq_pos(index: torch.Tensor, cu_seqlens: torch.Tensor):
    """(sequence id, position in sequence) of global token indices; tokens past the last sequence (padding) form one
    trailing pseudo-sequence so that each of them sees at least itself."""
    cu = cu_seqlens.long()
    seq = torch.bucketize(index, cu[1:], right=True)
    start = torch.cat([cu, cu[-1:]])[seq]
    return seq, index - start


def _partial(q, k, v, q_sp, k_sp, scale):
    """Attention of q against one K/V chunk: (normalised output fp32 [Tq, H, D], lse fp32 [Tq, H]; −inf / 0 where no key
    of the chunk is visible)."""
    rep = q.shape[1] // k.shape[1]
    kf, vf = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    vis = (q_sp[0][:, None] == k_sp[0][None, :]) & (k_sp[1][None, :] <= q_sp[1][:, None])
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    s = s.masked_fill(~vis[None], float("-inf"))
    lse = torch.logsumexp(s, -1)                                      # [H, Tq]
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(vis[None], p, torch.zeros_like(p))
    return torch.einsum("hqk,khd->qhd", p, vf), lse.t().contiguous()


def _merge(o, lse, o_new, lse_new):
    m = torch.logaddexp(lse, lse_new)
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    return o * torch.exp(lse - safe)[..., None] + o_new * torch.exp(lse_new - safe)[..., None], m


def _exchange(tensors, group, cp_size, cp_rank):
    """Send every tensor to the next rank of the ring and receive the previous rank's."""
    ranks = dist.get_process_group_ranks(group)
    nxt, prv = ranks[(cp_rank + 1) % cp_size], ranks[(cp_rank - 1) % cp_size]
    recv = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, prv, group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, total, group, cp_size, cp_rank, mode, scale):
        dev = q.device
        q_sp = _seq_pos(rank_token_index(total, cp_size, cp_rank, mode, dev), cu_seqlens)
        o = torch.zeros(q.shape, dtype=torch.float32, device=dev)
        lse = torch.full(q.shape[:2], float("-inf"), dtype=torch.float32, device=dev)
        kc, vc = k, v
        for step in range(cp_size):
            src = (cp_rank - step) % cp_size
            k_sp = _seq_pos(rank_token_index(total, cp_size, src, mode, dev), cu_seqlens)
            o_new, lse_new = _partial(q, kc, vc, q_sp, k_sp, scale)
            o, lse = _merge(o, lse, o_new, lse_new)
            if step + 1 < cp_size:
                kc, vc = _exchange([kc, vc], group, cp_size, cp_rank)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.cfg = (total, group, cp_size, cp_rank, mode, scale)
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_seqlens = ctx.saved_tensors
        total, group, cp_size, cp_rank, mode, scale = ctx.cfg
        dev = q.device
        rep = q.shape[1] // k.shape[1]
        q_sp = _seq_pos(rank_token_index(total, cp_size, cp_rank, mode, dev), cu_seqlens)
        dof, qf = do.float(), q.float()
        delta = (dof * o).sum(-1).t()                                   # [H, Tq]
        safe_lse = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).t()[..., None]
        dq = torch.zeros_like(qf)
        kc, vc = k.float(), v.float()
        dkc, dvc = torch.zeros_like(kc), torch.zeros_like(vc)
        for step in range(cp_size):
            src = (cp_rank - step) % cp_size
            k_sp = _seq_pos(rank_token_index(total, cp_size, src, mode, dev), cu_seqlens)
            kf, vf = kc.repeat_interleave(rep, 1), vc.repeat_interleave(rep, 1)
            vis = (q_sp[0][:, None] == k_sp[0][None, :]) & (k_sp[1][None, :] <= q_sp[1][:, None])
            s = torch.einsum("qhd,khd->hqk", qf, kf) * scale
            p = torch.where(vis[None], torch.exp(s - safe_lse), torch.zeros_like(s))
            dv = torch.einsum("hqk,qhd->khd", p, dof)
            dp = torch.einsum("qhd,khd->hqk", dof, vf)
            ds = p * (dp - delta[..., None]) * scale
            dq += torch.einsum("hqk,khd->qhd", ds, kf)
            dk = torch.einsum("hqk,qhd->khd", ds, qf)
            Tk, Hk = kc.shape[0], kc.shape[1]
            dkc += dk.view(Tk, Hk, rep, -1).sum(2)
            dvc += dv.view(Tk, Hk, rep, -1).sum(2)
            # the chunk and its gradient accumulators move on; after cp steps they are back at their owner
            kc, vc, dkc, dvc = _exchange([kc, vc, dkc, dvc], group, cp_size, cp_rank)
        return dq.to(q.dtype), dkc.to(k.dtype), dvc.to(v.dtype), None, None, None, None, None, None, None


def hierarchical_attention(q, k, v, cu_seqlens, ps, scale: float | None = None):
    """`a2a+p2p` context parallelism (the reference takes it from Megatron's hierarchical CP): inside an all-to-all group
    the members swap their sequence slices for head groups, so each holds the whole ring piece for H / a2a heads; K/V then
    travel round the ring of p2p members; the inverse all-to-all restores the sequence sharding."""
    from . import cp as _cp

    a, r = ps.cp_a2a_size, ps.cp_p2p_size
    total = q.shape[0] * ps.cp_size
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if a > 1:
        q, k, v = (_cp._SeqToHeads.apply(t.contiguous(), ps.cp_a2a_group, a) for t in (q, k, v))
    if r > 1:
        o = _RingAttention.apply(q, k, v, cu_seqlens, total, ps.cp_p2p_group, r, ps.cp_rank // a, "zigzag", scale)
    else:                                  # a ring of one: the all-to-all group holds the whole batch (plain Ulysses)
        from .. import ops

        o = ops.attention_varlen(q, k, v, cu_seqlens, int((cu_seqlens[1:] - cu_seqlens[:-1]).max()))
    return _cp._HeadsToSeq.apply(o.contiguous(), ps.cp_a2a_group, a) if a > 1 else o


def ring_attention(q, k, v, cu_seqlens, ps, scale: float | None = None):
    """q [Tl, Hq, D], k/v [Tl, Hkv, D]: this rank's tokens (`token_index` layout) → attention output [Tl, Hq, D]."""
    total = q.shape[0] * ps.cp_size
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _RingAttention.apply(q, k, v, cu_seqlens, total, ps.cp_group, ps.cp_size, ps.cp_rank, layout_mode(ps), scale)


class _AllGatherTokens(torch.autograd.Function):
    """Concatenate the ranks' token chunks (rank order); the gradient is reduce-scattered back."""

    @staticmethod
    def forward(ctx, x, group, cp_size, cp_rank):
        parts = [torch.empty_like(x) for _ in range(cp_size)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.cfg = (group, cp_size, cp_rank, x.shape[0])
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        group, cp_size, cp_rank, n = ctx.cfg
        g = g.contiguous()
        dist.all_reduce(g, group=group)
        return g[cp_rank * n:(cp_rank + 1) * n], None, None, None


def allgather_attention(q, k, v, cu_seqlens, ps, scale: float | None = None):
    """All-gather CP: every rank attends from its queries to the gathered K/V of the whole packed batch."""
    total = q.shape[0] * ps.cp_size
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    mode, dev = layout_mode(ps), q.device
    kf = _AllGatherTokens.apply(k, ps.cp_group, ps.cp_size, ps.cp_rank)
    vf = _AllGatherTokens.apply(v, ps.cp_group, ps.cp_size, ps.cp_rank)
    k_index = torch.cat([rank_token_index(total, ps.cp_size, r, mode, dev) for r in range(ps.cp_size)])
    q_sp = _seq_pos(rank_token_index(total, ps.cp_size, ps.cp_rank, mode, dev), cu_seqlens)
    o, _ = _partial(q, kf, vf, q_sp, _seq_pos(k_index, cu_seqlens), scale)
    return o.to(q.dtype)
