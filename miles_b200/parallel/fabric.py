"""NVLink fabric: symmetric buffers, peer pointer tables, flag barriers, and the fused compute+collective ops.

Every rank of one NVSwitch box allocates the same sequence of device buffers with plain `cudaMalloc`, exports an
IPC handle for each and maps every peer's buffer (`Fabric.alloc`).  A symmetric buffer therefore has one device
address per rank, usable from kernels on this GPU with ordinary loads and stores over NVLink.  Synchronisation is a
flag exchange kernel (system-scope release/acquire, waits bounded at one second, failures raise the device error
flag).  Nothing here uses TMA or cluster multicast on peer memory.

Fused paths built on it (kernels in `ops/csrc/comm.cu` and `ops/csrc/gemm_comm.cu`):
  * `moe_dispatch_combine`   expert-parallel dispatch → grouped tcgen05 GEMMs → return, no host synchronisation
  * `fused_optimizer_step`   gradient reduce-scatter (peer loads) + clip + AdamW + parameter all-gather (peer stores)
  * `allreduce_add_rmsnorm`  rollout TP all-reduce fused with residual add + RMSNorm
  * `ag_gemm` / `gemm_rs`    sequence-parallel all-gather → GEMM and GEMM → reduce-scatter
  * `vocab_logprob`          vocab-parallel log-prob / entropy with the max / sum merge over peers' statistics
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

# barrier channels (one flag row each)
CH_WORLD, CH_TP, CH_EP, CH_DP, CH_EP2, CH_TP2, CH_SYNC = 0, 1, 2, 3, 4, 5, 6
NUM_CHANNELS = 16


@dataclass
class Sym:
    """One symmetric allocation: the local tensor and every rank's mapping of it."""

    local: torch.Tensor                 # uint8 view of this rank's buffer
    views: list[torch.Tensor]           # uint8 tensors, one per world rank (peer memory for r != rank)
    nbytes: int

    def ptrs(self, ranks: list[int], offset_bytes: int = 0) -> torch.Tensor:
        return torch.tensor([self.views[r].data_ptr() + offset_bytes for r in ranks], dtype=torch.int64)


class Fabric:
    def __init__(self, ps, device: torch.device):
        from ..ops import cuda as K

        self.K = K
        self.C = K.C
        self.ps = ps
        self.rank, self.world = ps.rank, ps.world_size
        self.device = device
        self.syms: list[Sym] = []
        self._by_ptr: dict[int, tuple[Sym, int]] = {}
        self.err = self.C.error_flag(torch.empty(0, device=device))
        self.flags = self._alloc_sym(NUM_CHANNELS * 8 * 4)
        self.epochs = torch.zeros(NUM_CHANNELS, dtype=torch.int32, device=device)
        self._flag_ptrs: dict[tuple, torch.Tensor] = {}
        self._moe: dict[tuple, Any] = {}
        self._scratch: dict[str, Any] = {}
        self.configure()

    def configure(self, wait_ns: int | None = None):
        """Tell the peer-memory kernels where the error flag lives (so that, once it is raised, they return instead of
        consuming what a timed-out wait was guarding) and how long a wait on a peer may poll.  The limit defaults to
        `MILES_PEER_WAIT_MS` (5000 ms): long enough for host skew between ranks inside a phase, short enough that a lost
        peer ends the step with an error instead of a hang."""
        import os

        if wait_ns is None:
            wait_ns = int(float(os.environ.get("MILES_PEER_WAIT_MS", "5000")) * 1e6)
        self.wait_ns = int(wait_ns)
        self.C.fabric_configure(self.err, self.wait_ns)

    def phase_barrier(self, group=None):
        """Host-side rendezvous (NCCL / gloo) at a phase boundary — start of a rollout, of a train step, of a weight
        update — so that rank skew accumulated on the host (data conversion, garbage collection, checkpoint writes) is
        absorbed here, where waiting is unbounded and cheap, and not inside a kernel's bounded wait."""
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.barrier(group=group)

    def clear_error(self):
        self.err.zero_()

    @staticmethod
    def create(ps) -> "Fabric":
        dev = torch.device("cuda", torch.cuda.current_device())
        assert ps.world_size <= 8, "the fabric spans one NVSwitch box (≤ 8 GPUs)"
        return Fabric(ps, dev)

    # ---- symmetric allocation ------------------------------------------------------------------
    def _alloc_sym(self, nbytes: int) -> Sym:
        nbytes = (int(nbytes) + 255) // 256 * 256
        local, handle = self.C.fabric_alloc(nbytes, self.device.index)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, bytes(handle))
        views = []
        for r in range(self.world):
            views.append(local if r == self.rank else self.C.fabric_open(handles[r], nbytes, self.device.index))
        sym = Sym(local, views, nbytes)
        self.syms.append(sym)
        self._by_ptr[local.data_ptr()] = (sym, 0)
        dist.barrier()
        return sym

    def alloc(self, numel: int, dtype: torch.dtype, tag: str = "") -> torch.Tensor:
        """Collective: every rank must call with the same arguments in the same order. Returns the local tensor."""
        esize = torch.empty((), dtype=dtype).element_size()
        sym = self._alloc_sym(numel * esize)
        t = sym.local[: numel * esize].view(dtype)
        t._symmetric = True
        self._by_ptr[t.data_ptr()] = (sym, 0)
        return t

    def sym_of(self, t: torch.Tensor) -> tuple[Sym, int]:
        """(allocation, byte offset) of a tensor that lives inside a symmetric buffer."""
        p = t.data_ptr()
        if p in self._by_ptr:
            return self._by_ptr[p]
        for sym in self.syms:
            base = sym.local.data_ptr()
            if base <= p < base + sym.nbytes:
                return sym, p - base
        raise KeyError("tensor is not in symmetric memory")

    def peer_ptrs(self, t: torch.Tensor, ranks: list[int]) -> torch.Tensor:
        sym, off = self.sym_of(t)
        return sym.ptrs(ranks, off)

    # ---- barrier ----------------------------------------------------------------------------------
    def barrier(self, ranks: list[int], channel: int):
        """Cross-rank barrier among `ranks` (global ranks, in group order) enqueued on the current stream."""
        key = (tuple(ranks), channel)
        if key not in self._flag_ptrs:
            self._flag_ptrs[key] = self.flags.ptrs(ranks)
        self.C.barrier(self._flag_ptrs[key], ranks.index(self.rank), len(ranks), channel, self.epochs, self.err)

    def check(self):
        code = int(self.err.item())
        if code:
            raise RuntimeError(f"fabric kernel raised error flag {code} (bounded wait expired or receive buffer overflow)")

    def scratch(self, name: str, numel: int, dtype) -> torch.Tensor:
        """Cached symmetric scratch buffer, grown (collectively) on demand."""
        cur = self._scratch.get(name)
        if cur is None or cur.numel() < numel or cur.dtype != dtype:
            cur = self.alloc(max(numel, 1), dtype, tag=name)
            self._scratch[name] = cur
        return cur

    # ---- fused ops (implemented in sibling modules to keep this file small) -------------------------
    def moe_dispatch_combine(self, x, w13, w2, topk_w, topk_idx, num_experts, ps):
        from .ep_fused import fused_moe

        return fused_moe(self, x, w13, w2, topk_w, topk_idx, num_experts, ps)

    def allreduce_add_rmsnorm(self, partial, residual, w, eps, ps):
        from .tp_fused import allreduce_add_rmsnorm

        return allreduce_add_rmsnorm(self, partial, residual, w, eps, ps)

    def ag_gemm(self, x, w, ps):
        from .tp_fused import ag_gemm

        return ag_gemm(self, x, w, ps)

    def ag_gemm_dgrad(self, gy, w, ps):
        from .tp_fused import ag_gemm_dgrad

        return ag_gemm_dgrad(self, gy, w, ps)

    def gemm_rs(self, x, w, ps):
        from .tp_fused import gemm_rs

        return gemm_rs(self, x, w, ps)

    def reduce_scatter(self, x, ps):
        from .tp_fused import reduce_scatter

        return reduce_scatter(self, x, ps)

    def vocab_logprob(self, hidden, w, targets, temperature, with_entropy, ps):
        from .tp_fused import vocab_logprob

        return vocab_logprob(self, hidden, w, targets, temperature, with_entropy, ps)
