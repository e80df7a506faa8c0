"""Vocab-parallel log-prob / entropy over the fabric.

Each TP rank streams its vocabulary shard in chunks through the tcgen05 GEMM and folds every chunk into per-row
statistics {max, Σexp, Σexp·z, target z} (never materialising [tokens, vocab] logits); the per-rank statistics live
in symmetric memory and one small kernel merges all ranks' rows by peer loads after a flag barrier.  This replaces the
two/three TP all-reduces of Megatron's `fused_vocab_parallel_cross_entropy` and the reference's `_VocabParallelEntropy`
(miles/backends/training_utils/loss/hub/math_utils.py:297-310, 423-459).  Backward forms d logits per chunk from the
saved global log-sum-exp, accumulates dH in fp32 and reduces dH over the TP group with peer loads.
"""
from __future__ import annotations

import torch

from ..ops.cuda import BF16, _c, gemm_nt, gemm_tn
from ..ops.cuda_more import _VOCAB_CHUNK
from .fabric import CH_TP2


class _FusedVocabLogProb(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, w, targets, temperature, with_entropy, fab, ps):
        C = fab.C
        R, H = hidden.shape
        Vl = w.shape[0]
        ranks = ps.tp_ranks
        hidden = _c(hidden)
        tg = _c(targets.to(torch.int64)) - ps.tp_rank * Vl     # shard-local target ids (out of range on other ranks)
        inv_t = 1.0 / temperature
        par = fab._scratch.get("vstats.parity", 0)
        fab._scratch["vstats.parity"] = par ^ 1
        stats = fab.scratch(f"vstats.{par}", max(R, 1) * 4, torch.float32)[: R * 4].view(R, 4)
        for ci, v0 in enumerate(range(0, Vl, _VOCAB_CHUNK)):
            v1 = min(Vl, v0 + _VOCAB_CHUNK)
            logits = gemm_nt(hidden, w[v0:v1], out_dtype=torch.float32)
            C.logit_stats(logits, tg, stats, v0, inv_t, ci == 0)
        fab.barrier(ranks, CH_TP2)
        logp = torch.empty(R, dtype=torch.float32, device=hidden.device)
        ent = torch.empty(R, dtype=torch.float32, device=hidden.device)
        lse = torch.empty(R, dtype=torch.float32, device=hidden.device)
        C.stats_merge(fab.peer_ptrs(stats, ranks), len(ranks), logp, ent, lse)
        ctx.save_for_backward(hidden, w, tg, lse, ent)
        ctx.inv_t, ctx.with_entropy, ctx.fab, ctx.ps = inv_t, with_entropy, fab, ps
        return logp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, w, tg, lse, ent = ctx.saved_tensors
        fab, ps = ctx.fab, ctx.ps
        C = fab.C
        R, H = hidden.shape
        Vl = w.shape[0]
        g_lp = _c(g_lp.float()) if g_lp is not None else None
        g_ent = _c(g_ent.float()) if (g_ent is not None and ctx.with_entropy) else None
        dh = torch.zeros(R, H, dtype=torch.float32, device=hidden.device)
        dw = torch.empty_like(w)
        for v0 in range(0, Vl, _VOCAB_CHUNK):
            v1 = min(Vl, v0 + _VOCAB_CHUNK)
            logits = gemm_nt(hidden, w[v0:v1], out_dtype=torch.float32)
            dl = torch.empty(R, v1 - v0, dtype=BF16, device=hidden.device)
            C.logit_grad(logits, tg, lse, ent if g_ent is not None else None, g_lp, g_ent, dl, v0, ctx.inv_t)
            C.gemm(dl, w[v0:v1], dh, R, H, v1 - v0, v1 - v0, H, H, False, True, True, None, 0)
            gemm_tn(dl, hidden, out=dw[v0:v1])
        # dH is a partial sum over vocabulary shards: all-reduce it over the TP group (peer loads)
        from .tp_fused import _stage

        dhb = dh.to(hidden.dtype)
        staged = _stage(fab, "vdh", dhb, "vdh.parity")
        fab.barrier(ps.tp_ranks, CH_TP2)
        out = torch.empty_like(dhb)
        C.sum_rows(fab.peer_ptrs(staged, ps.tp_ranks), len(ps.tp_ranks), out)
        return out, dw, None, None, None, None, None


def fused_vocab_logprob(fab, hidden, w, targets, temperature, with_entropy, ps):
    if hidden.dtype != BF16:
        from .tp import _VocabParallelLogProb

        logp, ent = _VocabParallelLogProb.apply(hidden, w, targets, temperature, with_entropy, ps)
        return logp, (ent if with_entropy else None)
    logp, ent = _FusedVocabLogProb.apply(hidden, w, targets, float(temperature), bool(with_entropy), fab, ps)
    return logp, (ent if with_entropy else None)
