"""Expert parallelism: dispatch → local experts → combine.

Tokens are routed to the rank that owns each selected expert (contiguous expert ranges per EP rank),
run through that rank's experts and returned weighted by the gate — the "alltoall" token dispatcher
the reference forces for MoE (miles/utils/arguments.py:2857-2862; Megatron `--moe-token-dispatcher-type
alltoall`, scripts/models/qwen3-30B-A3B.py:35-43).

Executions:
* CUDA + fabric + `ps.fused`: `fabric.moe_dispatch_combine` — fused kernels that write token rows
  straight into the owners' receive buffers over NVLink (per-peer counters, bounded waits), run the
  tcgen05 grouped GEMMs, and push weighted results back into the source rank's output rows;
* otherwise `torch.distributed.all_to_all_single` with variable splits (NCCL on CUDA = the baseline,
  gloo on CPU for the multi-process tests), differentiable through `_AllToAll`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops


class _AllToAll(torch.autograd.Function):
    """Variable-split all-to-all over dim 0; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, group):
        ctx.group, ctx.send_counts, ctx.recv_counts = group, send_counts, recv_counts
        out = torch.empty((sum(recv_counts),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((sum(ctx.send_counts),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send_counts,
                               input_split_sizes=ctx.recv_counts, group=ctx.group)
        return out, None, None, None


def _exchange_counts(send_counts: torch.Tensor, group) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def expert_parallel_ffn(x, w13, w2, topk_w, topk_idx, num_experts: int, ps):
    """x [T,H]; w13 [E_local,2F,H]; w2 [E_local,H,F]; topk_w fp32 [T,k]; topk_idx int [T,k] (global ids)."""
    if x.is_cuda and ps.fabric is not None and ps.fused:
        return ps.fabric.moe_dispatch_combine(x, w13, w2, topk_w, topk_idx, num_experts, ps)
    T, H = x.shape
    k = topk_idx.shape[1]
    e_local = num_experts // ps.ep_size
    flat_e = topk_idx.reshape(-1).long()                      # [T·k]
    dest = flat_e // e_local
    order = torch.argsort(dest, stable=True)                  # group (token, slot) pairs by destination rank
    tok = (order // k)
    send_x = x.index_select(0, tok)                           # autograd: scatter-add in backward
    send_e = (flat_e[order] % e_local).to(torch.int32)
    send_counts_t = torch.bincount(dest, minlength=ps.ep_size).to(torch.int64)
    recv_counts_t = _exchange_counts(send_counts_t, ps.ep_group)
    send_counts, recv_counts = send_counts_t.tolist(), recv_counts_t.tolist()
    recv_x = _AllToAll.apply(send_x, send_counts, recv_counts, ps.ep_group)
    recv_e = torch.empty(sum(recv_counts), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_e, send_e, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                           group=ps.ep_group)
    if recv_x.shape[0] > 0:
        ones = torch.ones(recv_x.shape[0], 1, dtype=torch.float32, device=x.device)
        y_recv = ops.moe_ffn(recv_x, w13, w2, ones, recv_e[:, None])
    else:
        # keep the autograd graph (and the backward all-to-all) alive on ranks that received nothing
        y_recv = recv_x + 0.0 * (w13.sum() + w2.sum()).to(recv_x.dtype)
    back = _AllToAll.apply(y_recv, recv_counts, send_counts, ps.ep_group)   # rows in `order` order
    wflat = topk_w.reshape(-1)[order].to(torch.float32)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out = out.index_add(0, tok, back.float() * wflat[:, None])
    return out.to(x.dtype)
