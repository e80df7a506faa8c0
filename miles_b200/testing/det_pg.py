"""Deterministic in-process "process group": N ranks as threads of one process.

For tests of host-side logic that is written against collectives (metric reduction, micro-batch count agreement,
membership consensus, weight-update session framing) without spawning processes; the reference ships a deterministic
process group among its test utilities for the same purpose (miles/utils/test_utils/*).  Reductions always add in rank
order 0..N−1, so results are bit-reproducible run to run and independent of thread scheduling.

    world = LocalWorld(4)
    results = world.run(lambda pg: pg.all_reduce(torch.tensor([float(pg.rank)])))
"""
from __future__ import annotations

import threading
from typing import Any, Callable

import torch


class _Shared:
    def __init__(self, n: int):
        self.n = n
        self.barrier = threading.Barrier(n)
        self.slots: list[Any] = [None] * n
        self.calls: list[str] = []
        self.lock = threading.Lock()


class LocalPG:
    def __init__(self, rank: int, shared: _Shared):
        self.rank, self.world_size, self._s = rank, shared.n, shared

    def _exchange(self, value, name: str) -> list:
        s = self._s
        s.slots[self.rank] = value
        s.barrier.wait()
        got = list(s.slots)
        if self.rank == 0:
            with s.lock:
                s.calls.append(name)
        s.barrier.wait()                      # nobody overwrites a slot before everyone has read
        return got

    def barrier(self):
        self._exchange(None, "barrier")

    def all_gather_object(self, obj) -> list:
        return self._exchange(obj, "all_gather_object")

    def all_gather(self, t: torch.Tensor) -> list[torch.Tensor]:
        return [x.clone() for x in self._exchange(t.detach().clone(), "all_gather")]

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        parts = self._exchange(t.detach().clone(), f"all_reduce_{op}")
        acc = parts[0].clone()
        for p in parts[1:]:                   # fixed order → deterministic rounding
            acc = acc + p if op == "sum" else (torch.maximum(acc, p) if op == "max" else torch.minimum(acc, p))
        t.copy_(acc)
        return t

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        parts = self._exchange(t.detach().clone() if self.rank == src else None, "broadcast")
        t.copy_(parts[src])
        return t

    def broadcast_object(self, obj, src: int = 0):
        return self._exchange(obj if self.rank == src else None, "broadcast_object")[src]

    def all_to_all(self, chunks: list[torch.Tensor]) -> list[torch.Tensor]:
        assert len(chunks) == self.world_size
        everyone = self._exchange([c.detach().clone() for c in chunks], "all_to_all")
        return [everyone[src][self.rank].clone() for src in range(self.world_size)]

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        full = self.all_reduce(t.clone())
        return full.chunk(self.world_size, dim=0)[self.rank].clone()


class LocalWorld:
    def __init__(self, world_size: int):
        self.world_size = world_size
        self.shared = _Shared(world_size)

    def run(self, fn: Callable[[LocalPG], Any], timeout: float = 60.0) -> list:
        results: list[Any] = [None] * self.world_size
        errors: list[BaseException | None] = [None] * self.world_size

        def body(r):
            try:
                results[r] = fn(LocalPG(r, self.shared))
            except BaseException as e:
                errors[r] = e
                self.shared.barrier.abort()   # release peers blocked in a collective

        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.world_size)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout)
        first = next((e for e in errors if e is not None and not isinstance(e, threading.BrokenBarrierError)), None)
        if first is not None:
            raise first
        if any(t.is_alive() for t in threads):
            raise TimeoutError("a rank did not finish")
        return results

    @property
    def call_log(self) -> list[str]:
        return list(self.shared.calls)
