"""Worker providers: where the cells of a pool come from and how to reach them.

  `LocalProcessProvider`   cells are processes this job launched through the `WorkerManager`
  `StaticWorkerProvider`   cells run elsewhere at addresses given up front (a deployment made by other tooling)
  `RegistrationHub`        cells announce themselves: reporters post snapshots of the cells they watch; a reporter that
                           stops posting is dropped with its cells after a time-to-live (see registration.py)

All of them answer the same questions — list the cells with their workers' addresses, generation and liveness; watch
for changes — so the controllers above do not care which is in use (`--worker-provider`).

Reference: miles/utils/workers/worker_provider/base.py:13-53 (CellInfo, BaseWorkerProvider), static.py:25-104,
ray.py:17-72, worker_info.py, naming.py.
"""
from __future__ import annotations

import asyncio
import socket
from dataclasses import dataclass, field, replace
from typing import Awaitable, Callable


@dataclass(frozen=True)
class WorkerInfo:
    name: str
    pool: str
    cell_id: str
    index: int                                   # within the cell
    generation: int
    host: str = "127.0.0.1"
    ports: tuple = ()                            # ((port name, number), …)
    pid: int | None = None
    worker_class: str | None = None              # set for RPC-served python objects

    def port(self, name: str = "port") -> int:
        return dict(self.ports)[name]

    def url(self, name: str = "port") -> str:
        return f"http://{self.host}:{self.port(name)}"


@dataclass(frozen=True)
class CellInfo:
    cell_id: str
    pool: str
    generation: int
    alive: bool
    workers: tuple = ()


def worker_name(pool: str, cell: int, index: int) -> str:
    return f"{pool}-c{cell}-w{index}"


def cell_name(pool: str, cell: int) -> str:
    return f"{pool}-c{cell}"


CellReconcileFn = Callable[[str, "CellInfo | None"], Awaitable[None]]


class BaseWorkerProvider:
    async def init(self) -> None:
        pass

    async def list_cells(self) -> dict[str, CellInfo]:
        raise NotImplementedError

    async def get_addrs(self, name: str) -> WorkerInfo:
        for c in (await self.list_cells()).values():
            for w in c.workers:
                if w.name == name:
                    return w
        raise KeyError(name)

    async def get_worker_infos(self, cell_ids: list[str]) -> list[list[WorkerInfo]]:
        cells = await self.list_cells()
        return [list(cells[c].workers) if c in cells else [] for c in cell_ids]

    def expected_num_cells(self, pool: str) -> int | None:
        return None

    async def watch_cells(self, reconcile: CellReconcileFn, interval: float = 2.0):
        """Call `reconcile(cell_id, info | None)` for every change; returns an async stop function."""
        from .reconcile import PollingReconcileLoop

        return await PollingReconcileLoop(self.list_cells, interval).start(reconcile)


def tcp_alive(host: str, port: int, timeout: float = 0.5) -> bool:
    try:
        with socket.create_connection((host, port), timeout=timeout):
            return True
    except OSError:
        return False


def parse_host_port(addr: str) -> tuple[str, int]:
    addr = addr.split("://", 1)[-1].rstrip("/")
    host, _, port = addr.rpartition(":")
    assert host and port.isdigit(), f"expected host:port, got {addr!r}"
    return host, int(port)


class StaticWorkerProvider(BaseWorkerProvider):
    """One single-worker cell per address; a cell is alive while its port accepts connections."""

    def __init__(self, pool: str, addrs: list[str], worker_class: str | None = None, probe=tcp_alive):
        self.pool, self.probe = pool, probe
        self.workers = []
        for i, a in enumerate(addrs):
            h, p = parse_host_port(a)
            self.workers.append(WorkerInfo(worker_name(pool, i, 0), pool, cell_name(pool, i), 0, 0, h, (("port", p),), None, worker_class))

    async def list_cells(self):
        loop = asyncio.get_running_loop()
        alive = await asyncio.gather(*[loop.run_in_executor(None, self.probe, w.host, w.port()) for w in self.workers])
        return {w.cell_id: CellInfo(w.cell_id, self.pool, 0, bool(a), (w,)) for w, a in zip(self.workers, alive)}

    def expected_num_cells(self, pool):
        return len(self.workers) if pool == self.pool else None

    async def wait_ready(self, timeout: float = 120.0):
        end = asyncio.get_running_loop().time() + timeout
        while True:
            cells = await self.list_cells()
            if all(c.alive for c in cells.values()):
                return
            if asyncio.get_running_loop().time() > end:
                dead = [c for c, i in cells.items() if not i.alive]
                raise TimeoutError(f"static workers not reachable: {dead}")
            await asyncio.sleep(0.5)


class LocalProcessProvider(BaseWorkerProvider):
    def __init__(self, manager):
        self.manager = manager

    async def list_cells(self):
        return self.manager.get_cell_infos()

    def expected_num_cells(self, pool):
        return self.manager.num_cells(pool)


@dataclass
class CompositeProvider(BaseWorkerProvider):
    """Cells of several providers under one roof (launched engines + registered external ones)."""

    providers: list = field(default_factory=list)

    async def list_cells(self):
        out = {}
        for p in self.providers:
            out.update(await p.list_cells())
        return out

    def expected_num_cells(self, pool):
        ns = [p.expected_num_cells(pool) for p in self.providers]
        ns = [n for n in ns if n is not None]
        return sum(ns) if ns else None


def with_generation(info: CellInfo, generation: int) -> CellInfo:
    return replace(info, generation=generation, workers=tuple(replace(w, generation=generation) for w in info.workers))
