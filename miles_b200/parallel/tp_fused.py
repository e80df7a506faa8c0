"""Tensor-parallel ops over the NVLink fabric.

  allreduce_add_rmsnorm   rollout TP: partial rows of attention-out / MLP-down are summed straight out of every peer's
                          buffer inside the residual-add + RMSNorm kernel (one-shot all-reduce, peer loads)
  ag_gemm                 sequence-parallel all-gather → column GEMM: ONE kernel, the A tiles of remote row blocks are
                          fetched from the peers' buffers by the GEMM's own TMA producer as it reaches them
  gemm_rs                 row GEMM → reduce-scatter: ONE kernel, finished partial tiles are published per destination
                          and every rank sums its own row block out of the peers' partial buffers
  reduce_scatter          reduce-scatter of an existing tensor (backward of ag_gemm) with peer loads
  vocab_logprob           vocab-parallel log-prob / entropy: local streaming statistics, merged over peers' statistics

Synchronisation is the fabric's flag barrier (bounded waits).  Staging buffers are double buffered so that a rank may
run one call ahead of its peers without overwriting data they still read.
"""
from __future__ import annotations

import torch

from ..ops.cuda import gemm_nn, gemm_nt, gemm_tn
from .fabric import CH_TP, CH_TP2


def _stage(fab, name: str, x: torch.Tensor, parity_key: str) -> torch.Tensor:
    """Copy x into a (double-buffered) symmetric staging buffer and return the staged view."""
    par = fab._scratch.get(parity_key, 0)
    fab._scratch[parity_key] = par ^ 1
    buf = fab.scratch(f"{name}.{par}", x.numel(), x.dtype)
    v = buf[: x.numel()].view(x.shape)
    v.copy_(x)
    return v


TWO_SHOT_MIN_BYTES = 1 << 20      # per-rank partial size from which the two-shot schedule moves fewer bytes over NVLink


def allreduce_add_rmsnorm(fab, partial, residual, w, eps, ps):
    """(y, new_residual) = add_rmsnorm(Σ_ranks partial, residual).  `partial` [T, H] bf16 on every TP rank.

    One-shot (decode-sized inputs): every rank reads all peers' rows inside the norm kernel — (tp−1)·T·H elements in,
    one barrier, one kernel.  Two-shot (prefill-sized inputs, tp ≥ 4, T divisible by tp): each rank sums ITS row block
    out of the peers' buffers, the reduced blocks are gathered with peer loads, the add + norm then runs on local data —
    2·(tp−1)/tp·T·H elements in, which at tp = 8 is a quarter of the one-shot traffic."""
    ranks = ps.tp_ranks
    tp = len(ranks)
    T, H = partial.shape
    staged = _stage(fab, "ar", partial.contiguous(), "ar.parity")
    if tp >= 4 and T % tp == 0 and partial.numel() * 2 >= TWO_SHOT_MIN_BYTES and (T // tp) * H % 8 == 0:
        from ..ops import add_rmsnorm

        n = T // tp
        fab.barrier(ranks, CH_TP)
        par = fab._scratch.get("ar2.parity", 0)
        fab._scratch["ar2.parity"] = par ^ 1
        red = fab.scratch(f"ar2.{par}", n * H, partial.dtype)[: n * H].view(n, H)
        sym, off = fab.sym_of(staged)
        fab.C.sum_rows(sym.ptrs(ranks, off + ps.tp_rank * n * H * partial.element_size()), tp, red)
        fab.barrier(ranks, CH_TP2)
        total = torch.empty_like(partial)
        fab.C.gather_rows(fab.peer_ptrs(red, ranks), tp, total)
        return add_rmsnorm(total, residual, w, eps)
    fab.barrier(ranks, CH_TP)
    y = torch.empty_like(partial)
    r = torch.empty_like(partial)
    fab.C.ar_add_rmsnorm(fab.peer_ptrs(staged, ranks), len(ranks), residual, w, y, r, eps)
    return y, r


def ag_gemm(fab, x, w, ps):
    """y [T, N/tp] = all_gather_seq(x [T/tp, K]) · wᵀ, returning (y, gathered x or None)."""
    from .gemm_comm import ag_gemm_fused

    return ag_gemm_fused(fab, x, w, ps)


def gemm_rs(fab, x, w, ps):
    """y [T/tp, N] = reduce_scatter_seq(x [T, K/tp] · wᵀ)."""
    from .gemm_comm import gemm_rs_fused

    return gemm_rs_fused(fab, x, w, ps)


def reduce_scatter(fab, x, ps):
    """out [T/tp, N] = Σ_ranks x[rank rows].  One-shot: every rank reads its row block from all peers."""
    ranks = ps.tp_ranks
    tp = len(ranks)
    T, N = x.shape
    n = T // tp
    staged = _stage(fab, "rs", x.contiguous(), "rs.parity")
    fab.barrier(ranks, CH_TP2)
    out = torch.empty(n, N, dtype=x.dtype, device=x.device)
    sym, off = fab.sym_of(staged)
    ptrs = sym.ptrs(ranks, off + ps.tp_rank * n * N * x.element_size())
    fab.C.sum_rows(ptrs, tp, out)
    return out


def ag_gemm_dgrad(fab, gy, w, ps):
    """Backward of the row-parallel linear: (gx [T, K/tp], gathered gy [T, N]) = (all_gather_seq(gy) · w, gathered gy)."""
    ranks = ps.tp_ranks
    tp = len(ranks)
    n, N = gy.shape
    staged = _stage(fab, "agd", gy.contiguous(), "agd.parity")
    fab.barrier(ranks, CH_TP)
    gyg = torch.empty(n * tp, N, dtype=gy.dtype, device=gy.device)
    fab.C.gather_rows(fab.peer_ptrs(staged, ranks), tp, gyg)
    return gemm_nn(gyg, w), gyg


def vocab_logprob(fab, hidden, w, targets, temperature, with_entropy, ps):
    from .vocab_fused import fused_vocab_logprob

    return fused_vocab_logprob(fab, hidden, w, targets, temperature, with_entropy, ps)
