"""Context parallelism: sequence sharding helpers and the Ulysses (all-to-all) attention layout.

The reference supports ring CP with zigzag slicing, Ulysses (`cp_comm_type == "a2a"`) and all-gather CP with contiguous
chunks (miles/backends/training_utils/data/context_parallel.py:13-471, data/rollout.py:233-297).  Here the trainer
shards every packed micro-batch into contiguous chunks of T/cp tokens; attention swaps the sharding from sequence to
heads with one all-to-all before the kernel and back after it (Ulysses), so the attention kernel itself is the
single-GPU one and sees whole sequences.  Over NVSwitch the all-to-all moves (1 − 1/cp) of q/k/v/o once per layer at
full bisection bandwidth, against cp − 1 ring steps of K/V for ring attention.

Also here: zigzag index helpers (for checkpoints / data laid out for ring CP), the differentiable gather that rebuilds
full per-token vectors (log-probs, entropy) from CP shards for sequence-level losses, and the loss-mask-weighted
"sum of sample means" used for metric reduction.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


# ---- chunking ------------------------------------------------------------------------------------------------

def chunk_bounds(total: int, cp_size: int, cp_rank: int) -> tuple[int, int]:
    """Contiguous chunk [lo, hi) of a length-`total` token axis (total must divide by cp_size)."""
    assert total % cp_size == 0, f"packed length {total} must be a multiple of cp_size {cp_size}"
    n = total // cp_size
    return cp_rank * n, (cp_rank + 1) * n


def zigzag_bounds(total: int, cp_size: int, cp_rank: int) -> list[tuple[int, int]]:
    """Ring-attention load balancing: the axis is cut into 2·cp pieces and rank r owns pieces r and 2·cp−1−r."""
    assert total % (2 * cp_size) == 0
    n = total // (2 * cp_size)
    a, b = cp_rank, 2 * cp_size - 1 - cp_rank
    return [(a * n, (a + 1) * n), (b * n, (b + 1) * n)]


def slice_with_cp(x: torch.Tensor, cp_size: int, cp_rank: int, mode: str = "contiguous", dim: int = 0) -> torch.Tensor:
    if cp_size == 1:
        return x
    if mode == "contiguous":
        lo, hi = chunk_bounds(x.shape[dim], cp_size, cp_rank)
        return x.narrow(dim, lo, hi - lo)
    parts = [x.narrow(dim, lo, hi - lo) for lo, hi in zigzag_bounds(x.shape[dim], cp_size, cp_rank)]
    return torch.cat(parts, dim=dim)


def zigzag_to_contiguous_index(total: int, cp_size: int) -> torch.Tensor:
    """Permutation p with concat_r(zigzag shard r)[p] == original order (redistribution between the two layouts)."""
    order = []
    for r in range(cp_size):
        for lo, hi in zigzag_bounds(total, cp_size, r):
            order.extend(range(lo, hi))
    inv = torch.empty(total, dtype=torch.long)
    inv[torch.tensor(order)] = torch.arange(total)
    return inv


# ---- differentiable collectives ------------------------------------------------------------------------------

class _AllReduceSumIdentityGrad(torch.autograd.Function):
    """Forward: sum over the CP group.  Backward: identity — each rank contributed a disjoint piece of the vector, every
    rank evaluates the same loss on the sum, and parameter gradients are later summed over the CP group."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def gather_from_cp(local_values: torch.Tensor, select: torch.Tensor, total: int, ps) -> torch.Tensor:
    """Place this rank's values at positions `select` (bool [total]) of a zero vector and sum over the CP group:
    every rank ends with the full vector, gradients flow to the local piece only."""
    full = torch.zeros(total, dtype=local_values.dtype, device=local_values.device)
    full = full.masked_scatter(select, local_values) if local_values.numel() else full + 0 * local_values.sum()
    if ps.cp_size == 1:
        return full
    return _AllReduceSumIdentityGrad.apply(full, ps.cp_group)


class _SeqToHeads(torch.autograd.Function):
    """[T/cp, H, D] sharded by sequence → [T, H/cp, D] sharded by heads (one all-to-all); backward is the inverse."""

    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        return _a2a_seq_to_heads(x, group, cp)

    @staticmethod
    def backward(ctx, g):
        return _a2a_heads_to_seq(g.contiguous(), ctx.group, ctx.cp), None, None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        return _a2a_heads_to_seq(x, group, cp)

    @staticmethod
    def backward(ctx, g):
        return _a2a_seq_to_heads(g.contiguous(), ctx.group, ctx.cp), None, None


def _a2a_seq_to_heads(x, group, cp):
    Tl, H, D = x.shape
    assert H % cp == 0, f"{H} heads do not divide by cp_size {cp}"
    send = x.reshape(Tl, cp, H // cp, D).permute(1, 0, 2, 3).contiguous()     # [cp, Tl, H/cp, D]: block j → rank j
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                           # block j = chunk j of my head group
    return recv.reshape(cp * Tl, H // cp, D)


def _a2a_heads_to_seq(x, group, cp):
    T, Hl, D = x.shape
    Tl = T // cp
    send = x.reshape(cp, Tl, Hl, D).contiguous()                              # block j = chunk j → rank j
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                           # block j = my chunk, head group j
    return recv.permute(1, 0, 2, 3).reshape(Tl, cp * Hl, D)


def seq_to_heads(x, ps):
    return x if ps.cp_size == 1 else _SeqToHeads.apply(x.contiguous(), ps.cp_group, ps.cp_size)


def heads_to_seq(x, ps):
    return x if ps.cp_size == 1 else _HeadsToSeq.apply(x.contiguous(), ps.cp_group, ps.cp_size)


# ---- reductions ------------------------------------------------------------------------------------------------

def sum_of_sample_mean(x: torch.Tensor, loss_mask: torch.Tensor, seq_ids: torch.Tensor, num_samples: int,
                       denominators: torch.Tensor | None = None) -> torch.Tensor:
    """Σ_samples (Σ_tokens x·mask / Σ_tokens mask): the default loss / metric reduction; `denominators` overrides the
    per-sample mask sums (siblings of one rollout share one)."""
    num = torch.zeros(num_samples, dtype=torch.float32, device=x.device).index_add_(0, seq_ids, (x * loss_mask).float())
    den = denominators if denominators is not None else \
        torch.zeros(num_samples, dtype=torch.float32, device=x.device).index_add_(0, seq_ids, loss_mask.float())
    return (num / den.clamp_min(1.0)).sum()
