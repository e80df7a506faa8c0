"""Independent data-parallel replicas ("cells") with a reconfigurable cross-cell gradient all-reduce.

Reference: miles/backends/megatron_utils/ft/indep_dp.py:23-193 and miles/ray/train/group.py:520-675.  With `--indep-dp`
every DP replica is its own training world; gradients are averaged across the replicas through a process group that
can be rebuilt when membership changes (torchft there, a TCPStore-rendezvoused group here), an intra-step consensus
(all-reduce MIN of an ok flag) decides whether every surviving cell commits the optimizer step, and a failed step is
discarded and retried on the remaining quorum.

Failure model on this code path: a cell stops between steps (its process raised, exited or was fenced by the
controller).  Survivors learn of it on the host — through the store's membership key, or because the next collective
raises after the short group timeout — never by waiting inside a device kernel.
"""
from __future__ import annotations

import datetime
import time

import torch
import torch.distributed as dist


class CellMembership:
    """Membership record in a key-value store: epoch counter + comma-separated list of live cell ids."""

    def __init__(self, store, prefix: str = "indep_dp"):
        self.store, self.prefix = store, prefix

    def publish(self, epoch: int, cells: list[int]):
        self.store.set(f"{self.prefix}/members/{epoch}", ",".join(str(c) for c in sorted(cells)))
        self.store.set(f"{self.prefix}/epoch", str(epoch))

    def current(self) -> tuple[int, list[int]]:
        epoch = int(self.store.get(f"{self.prefix}/epoch").decode())
        raw = self.store.get(f"{self.prefix}/members/{epoch}").decode()
        return epoch, [int(c) for c in raw.split(",") if c]

    def report_dead(self, cell: int):
        self.store.set(f"{self.prefix}/dead/{cell}", str(time.time()))

    def is_dead(self, cell: int) -> bool:
        return self.store.check([f"{self.prefix}/dead/{cell}"])


class IndepDP:
    """Cross-cell communicator of ONE rank position (rank r of every cell forms one group)."""

    def __init__(self, cell_id: int, host: str, port: int, *, backend: str = "gloo", timeout_s: float = 10.0,
                 is_store_master: bool = False, expected_cells: int = 1):
        self.cell_id, self.backend, self.timeout_s = cell_id, backend, timeout_s
        self.store = dist.TCPStore(host, port, None, is_master=is_store_master,
                                   timeout=datetime.timedelta(seconds=max(timeout_s, 30.0)), wait_for_workers=False)
        self.members = CellMembership(self.store)
        self.epoch = -1
        self.cells: list[int] = []
        self.pg = None
        self.expected_cells = expected_cells

    # ---- group (re)construction --------------------------------------------------------------------
    def configure(self, epoch: int, cells: list[int]):
        """Build the group of membership `epoch`.  Every live cell calls this with the same arguments."""
        cells = sorted(cells)
        assert self.cell_id in cells
        self.pg = None                                   # drop the old group before the new rendezvous
        store = dist.PrefixStore(f"indep_dp_pg_{epoch}", self.store)
        to = datetime.timedelta(seconds=self.timeout_s)
        rank, world = cells.index(self.cell_id), len(cells)
        if world == 1:
            self.pg = None
        elif self.backend == "nccl":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = to
            self.pg = dist.ProcessGroupNCCL(store, rank, world, opts)
        else:
            self.pg = dist.ProcessGroupGloo(store, rank, world, to)
        self.epoch, self.cells = epoch, cells

    def follow_membership(self):
        """Adopt the newest published membership if it differs from the current one."""
        epoch, cells = self.members.current()
        if epoch != self.epoch:
            self.configure(epoch, cells)
        return self.epoch

    # ---- collectives -----------------------------------------------------------------------------
    def _all_reduce(self, t: torch.Tensor, op):
        if self.pg is None:
            return
        opts = dist.AllreduceOptions()
        opts.reduceOp = op
        self.pg.allreduce([t], opts).wait()

    def all_reduce_grads(self, buckets: list[torch.Tensor], average: bool = True):
        """Sum each gradient bucket over the cells (then divide by the number of cells).  Raises on a dead peer."""
        for b in buckets:
            self._all_reduce(b, dist.ReduceOp.SUM)
            if average and len(self.cells) > 1:
                b.div_(len(self.cells))

    def consensus(self, ok: bool) -> bool:
        """True iff every live cell reports ok (all-reduce MIN): commit the step or discard it everywhere."""
        t = torch.tensor([1 if ok else 0], dtype=torch.int32)
        if self.backend == "nccl" and self.pg is not None:
            t = t.cuda()
        self._all_reduce(t, dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def step(self, buckets: list[torch.Tensor], local_ok: bool = True, max_retries: int = 3):
        """One fault-tolerant gradient exchange.  Returns (committed, cells that took part).

        A collective that raises (peer gone, timeout) makes the caller wait for the controller to publish a new
        membership, rebuild the group and retry on the saved gradients; the optimizer step of the failed attempt is
        never applied, so surviving cells stay bit-identical."""
        saved = [b.clone() for b in buckets]
        for attempt in range(max_retries + 1):
            try:
                self.all_reduce_grads(buckets)
                return self.consensus(local_ok), list(self.cells)
            except Exception:
                if attempt == max_retries:
                    raise
                for b, s in zip(buckets, saved):
                    b.copy_(s)
                self._wait_for_new_membership()
        return False, list(self.cells)

    def _wait_for_new_membership(self, poll_s: float = 0.05, limit_s: float = 60.0):
        t0 = time.time()
        while time.time() - t0 < limit_s:
            epoch, cells = self.members.current()
            if epoch != self.epoch and self.cell_id in cells:
                self.configure(epoch, cells)
                return
            time.sleep(poll_s)
        raise TimeoutError("no new cell membership was published after a failed collective")
