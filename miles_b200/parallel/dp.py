"""Fused data-parallel optimizer step over the NVLink fabric.

    barrier → reduce this rank's shard straight out of every peer's fp32 gradient buffer (+ Σg²)
            → one world all-reduce of the scalar Σg² (global clip norm)
            → AdamW on the shard, bf16 results stored into every peer's parameter buffer → barrier

The gradient buffers and parameter buffers of a reduction domain live in symmetric memory (allocated through the
fabric by `TrainActor._symmetric_allocator`), so the reduce-scatter is peer *loads* inside the reduction kernel and the
parameter all-gather is peer *stores* inside the Adam kernel; no NCCL bucket traffic and no staging copies.  This is
the role of Megatron's DDP bucket reduce-scatter + distributed optimizer + parameter all-gather in the reference
(miles/backends/megatron_utils/model.py:248-273, 639-642, 686-701).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .fabric import CH_DP


def _domain_ranks(d, ps):
    if d.name == "dense":
        return ps.dp_ranks if ps.cp_size == 1 else None
    return None  # expert domain: expert-data-parallel groups; fused only when edp == 1 (nothing to reduce)


def fused_step(opt, lr):
    ps = opt.ps
    fab = ps.fabric
    C = fab.C
    for d in opt.domains:
        if d.group_size > 1 and (_domain_ranks(d, ps) is None or not getattr(d.grad_buf, "_symmetric", False)):
            return None   # layout not covered: fall back to the collective path
    dev = opt.domains[0].param_buf.device
    sq = torch.zeros(1, dtype=torch.float32, device=dev)
    b1, b2 = opt.betas
    shards = []
    for d in opt.domains:
        lo, hi = d.shard
        if d.group_size > 1:
            ranks = _domain_ranks(d, ps)
            fab.barrier(ranks, CH_DP)
            nw = getattr(opt, "_tp_replicated_mask", {}).get(d.name)
            norm_w = (1.0 - nw) if (nw is not None and ps.tp_size > 1 and ps.tp_rank != 0) else None
            C.rs_reduce_sqnorm(fab.peer_ptrs(d.grad_buf, ranks), len(ranks), ranks.index(ps.rank), lo, hi, norm_w, sq)
        else:
            g = d.grad_buf[lo:hi]
            sq += (g * g).sum()
        shards.append(d.grad_buf[lo:hi])
    if ps.world_size > 1:
        dist.all_reduce(sq)   # every shard is owned by exactly one rank, so the sum is the global Σg²
    for d, g in zip(opt.domains, shards):
        lo, hi = d.shard
        if d.group_size > 1:
            ranks = _domain_ranks(d, ps)
            C.adam_allgather(d.master, g, d.exp_avg, d.exp_avg_sq, d.decay_mask, sq, float(opt.clip_grad or 0.0),
                             fab.peer_ptrs(d.param_buf, ranks), len(ranks), lo, lr, b1, b2, opt.eps, opt.weight_decay,
                             opt.step_count)
            fab.barrier(ranks, CH_DP)
        else:
            scale = torch.clamp(opt.clip_grad / (sq.sqrt() + 1e-6), max=1.0) if opt.clip_grad else 1.0
            fab.K.adamw_step_masked(d.master, g, d.exp_avg, d.exp_avg_sq, d.decay_mask, lr, b1, b2, opt.eps, opt.weight_decay,
                                    opt.step_count, scale, d.param_buf[lo:hi])
    return {"grad_norm": float(sq.sqrt().item())}
