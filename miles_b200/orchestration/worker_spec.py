"""Declarative worker pools, GPU slot placement and port allocation.

Reference: miles/utils/workers/worker_spec.py:20-166 (`ServeWorkerSpec`: a python class served as an actor / RPC
endpoint; `CommandWorkerSpec`: a shell command such as an engine server; `SchedulingSpec`: cells × workers × GPU
slots), miles/ray/placement_group.py:48-162 (bundles sorted by (node, GPU id); layout `max(train, rollout)` when
colocated else `train + rollout`) and the port allocation of miles/ray/specs/inference.py:292-424.

On one NVSwitch box a "placement group" is a list of (node, gpu) slots: the planner here assigns slots to pools, builds
each worker's environment (`CUDA_VISIBLE_DEVICES`, `RANK`, `WORLD_SIZE`, `MASTER_ADDR`, `MASTER_PORT`) and its command
line; `LocalLauncher` runs the plan as subprocesses (or as RPC-served python objects) on this machine.
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Any


@dataclass
class SchedulingSpec:
    num_cells: int = 1               # replicas of the pool
    workers_per_cell: int = 1
    gpus_per_worker: float = 1.0     # < 1 lets another pool share the GPU (colocated trainer + engine)


@dataclass
class ServeWorkerSpec:
    name: str
    target: str                      # "module.Class" constructed in the worker, served over RPC
    scheduling: SchedulingSpec = field(default_factory=SchedulingSpec)
    init_kwargs: dict = field(default_factory=dict)
    env: dict = field(default_factory=dict)
    concurrency: dict = field(default_factory=lambda: {"default": 1, "health": 2})


@dataclass
class CommandWorkerSpec:
    name: str
    command: list[str]               # may contain {port}, {rank}, {world_size}, {gpu_ids}, {master_port}
    scheduling: SchedulingSpec = field(default_factory=SchedulingSpec)
    env: dict = field(default_factory=dict)
    ports: list[str] = field(default_factory=lambda: ["port"])   # named ports to allocate per worker


@dataclass
class Slot:
    node: str
    gpu: int


@dataclass
class PlannedWorker:
    pool: str
    cell: int
    rank: int                        # rank within the cell
    global_rank: int                 # rank within the pool
    slots: list[Slot]
    env: dict
    command: list[str] | None
    ports: dict[str, int]
    spec: Any


def sorted_slots(nodes: dict[str, int]) -> list[Slot]:
    """All GPU slots ordered by (node, gpu id) — the order ranks are laid out in."""
    return [Slot(n, g) for n in sorted(nodes) for g in range(nodes[n])]


class PortAllocator:
    def __init__(self, base: int = 0, host: str = "127.0.0.1"):
        self.base, self.host = base, host
        self.given: set[int] = set()

    def get(self) -> int:
        if self.base:
            p = self.base
            while p in self.given or not self._free(p):
                p += 1
            self.base = p + 1
        else:
            with socket.socket() as s:
                s.bind((self.host, 0))
                p = s.getsockname()[1]
            while p in self.given:
                p += 1
        self.given.add(p)
        return p

    def _free(self, port: int) -> bool:
        with socket.socket() as s:
            try:
                s.bind((self.host, port))
                return True
            except OSError:
                return False


def plan(specs: list, nodes: dict[str, int], colocate: bool = False, ports: PortAllocator | None = None,
         master_addr: str = "127.0.0.1", first_slot: int = 0) -> list[PlannedWorker]:
    """Assign GPU slots to every worker of every pool.  `colocate`: pools overlap on the same slots (layout =
    max over pools), otherwise pools take consecutive disjoint slot ranges (layout = sum).  `first_slot`: slots before it
    belong to someone else (the trainer's ranks of a disaggregated job)."""
    ports = ports or PortAllocator()
    slots = sorted_slots(nodes)[first_slot:]
    out: list[PlannedWorker] = []
    cursor = 0
    for spec in specs:
        sch = spec.scheduling
        n_workers = sch.num_cells * sch.workers_per_cell
        per = max(1, int(round(sch.gpus_per_worker))) if sch.gpus_per_worker >= 1 else 1
        need = n_workers * per if sch.gpus_per_worker > 0 else 0
        start = 0 if colocate else cursor
        assert start + need <= len(slots), f"pool {spec.name} needs {need} GPU slots from {start}, only {len(slots)} exist"
        master_port = ports.get()
        for w in range(n_workers):
            mine = slots[start + w * per: start + (w + 1) * per] if need else []
            cell, rank = divmod(w, sch.workers_per_cell)
            wports = {p: ports.get() for p in getattr(spec, "ports", [])}
            env = {"RANK": str(rank), "WORLD_SIZE": str(sch.workers_per_cell), "LOCAL_RANK": str(mine[0].gpu if mine else 0),
                   "MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port + cell), "MILES_POOL": spec.name, "MILES_CELL": str(cell),
                   "CUDA_VISIBLE_DEVICES": ",".join(str(s.gpu) for s in mine), **{k: str(v) for k, v in spec.env.items()}}
            cmd = None
            if isinstance(spec, CommandWorkerSpec):
                fmt = dict(rank=rank, world_size=sch.workers_per_cell, gpu_ids=",".join(str(s.gpu) for s in mine), master_port=master_port + cell,
                           cell=cell, **wports)
                cmd = [c.format(**fmt) for c in spec.command]
            out.append(PlannedWorker(spec.name, cell, rank, w, mine, env, cmd, wports, spec))
        if not colocate:
            cursor += need
    return out


class LocalLauncher:
    """Run a plan on this machine: command workers as subprocesses, serve workers as RPC endpoints in subprocesses."""

    def __init__(self):
        self.procs: list[tuple[PlannedWorker, subprocess.Popen]] = []

    def launch(self, workers: list[PlannedWorker], dry_run: bool = False) -> list[dict]:
        described = []
        for w in workers:
            if isinstance(w.spec, CommandWorkerSpec):
                cmd = w.command
            else:
                port = w.ports.get("rpc") or PortAllocator().get()
                w.ports["rpc"] = port
                cmd = [sys.executable, "-m", "miles_b200.orchestration.worker_spec", "--serve", w.spec.target, "--port", str(port),
                       "--kwargs", repr(w.spec.init_kwargs)]
            described.append({"pool": w.pool, "cell": w.cell, "rank": w.rank, "cmd": cmd, "env": w.env, "ports": w.ports})
            if not dry_run:
                self.procs.append((w, subprocess.Popen(cmd, env={**os.environ, **w.env})))
        return described

    def stop(self):
        for _, p in self.procs:            # exact PIDs of the processes this launcher started
            if p.poll() is None:
                p.terminate()
        for _, p in self.procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()
        self.procs.clear()


def _serve_main():
    import argparse
    import ast
    import time

    from ..utils.misc import load_function
    from .rpc import RpcServer

    p = argparse.ArgumentParser()
    p.add_argument("--serve", required=True)
    p.add_argument("--port", type=int, required=True)
    p.add_argument("--kwargs", default="{}")
    a = p.parse_args()
    obj = load_function(a.serve)(**ast.literal_eval(a.kwargs))
    RpcServer(obj, concurrency={"default": 1, "health": 2}, groups={"ping": "health", "health": "health"}).start(a.port)
    while True:
        time.sleep(3600)


if __name__ == "__main__":
    _serve_main()
