"""Python side of the fused tensor-parallel GEMMs (`ops/csrc/gemm_comm.cu`)."""
from __future__ import annotations

import torch

from .fabric import CH_TP, CH_TP2

_CH_AG, _CH_RS = 8, 9   # dedicated flag rows; epochs are tracked here because these kernels take them as arguments


def _next_epoch(fab, ch: int) -> int:
    key = f"epoch.{ch}"
    e = fab._scratch.get(key, 0) + 1
    fab._scratch[key] = e
    return e


def _flag_ptrs(fab, ranks):
    key = (tuple(ranks), "raw")
    if key not in fab._flag_ptrs:
        fab._flag_ptrs[key] = fab.flags.ptrs(ranks)
    return fab._flag_ptrs[key]


def ag_gemm_fused(fab, x, w, ps):
    """y [T, N_local] = all_gather_seq(x [T/tp, K]) · wᵀ in one kernel. Returns (y, None).

    The symmetric buffer holds the whole gathered [T, K] matrix; this rank writes its own row block, the kernel's copy
    warps fill the others from the peers' buffers (each remote row crosses NVLink once) while the tensor-core tiles of
    this rank's own rows already run."""
    ranks = ps.tp_ranks
    tp = len(ranks)
    n, K = x.shape
    assert n % 128 == 0, "sequence-parallel chunks are padded to 128 rows"
    par = fab._scratch.get("agx.parity", 0)
    fab._scratch["agx.parity"] = par ^ 1
    buf = fab.scratch(f"agx.{par}", n * tp * K, x.dtype)
    xg = buf[: n * tp * K].view(n * tp, K)
    xg[ps.tp_rank * n:(ps.tp_rank + 1) * n].copy_(x)
    counters = fab._scratch.get("ag.counters")
    if counters is None or counters.numel() * 128 < n * tp:
        counters = torch.zeros(max(1024, n * tp // 128), dtype=torch.int32, device=x.device)
        fab._scratch["ag.counters"] = counters
    y = torch.empty(n * tp, w.shape[0], dtype=x.dtype, device=x.device)
    fab.C.ag_gemm(fab.peer_ptrs(xg, ranks), w.contiguous(), y, counters, n, ps.tp_rank, tp, _flag_ptrs(fab, ranks), _CH_AG,
                  _next_epoch(fab, _CH_AG), fab.err)
    return y, None


def gemm_rs_fused(fab, x, w, ps):
    """y [T/tp, N] = reduce_scatter_seq(x [T, K_local] · wᵀ) in one kernel.  The symmetric buffer is `tp` slots of
    [T/tp, N]: slot r of rank d receives rank r's partial rows for d, pushed from r's GEMM epilogue."""
    ranks = ps.tp_ranks
    tp = len(ranks)
    T, K = x.shape
    N = w.shape[0]
    assert T % (128 * tp) == 0
    par = fab._scratch.get("rsp.parity", 0)
    fab._scratch["rsp.parity"] = par ^ 1
    partial = fab.scratch(f"rsp.{par}", T * N, x.dtype)
    counters = fab._scratch.get("rs.counters")
    if counters is None:
        counters = torch.zeros(8, dtype=torch.int32, device=x.device)
        fab._scratch["rs.counters"] = counters
    out = torch.empty(T // tp, N, dtype=x.dtype, device=x.device)
    fab.C.gemm_rs(x.contiguous(), w.contiguous(), fab.peer_ptrs(partial, ranks), out, counters, ps.tp_rank, tp, _flag_ptrs(fab, ranks),
                  _CH_RS, _next_epoch(fab, _CH_RS), fab.err)
    return out
