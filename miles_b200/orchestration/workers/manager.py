"""WorkerManager: pools → cells → worker processes on this machine, with generations.

`launch(specs, nodes)` plans GPU slots and ports (`worker_spec.plan`) and starts every worker; a CELL is the unit of
failure and restart: when any of its processes has exited the cell is dead, `restart_cell` stops what is left and
starts all of its workers again under generation + 1, so that handles made for an older generation can be told apart
(`get_worker(name, expected_generation=…)` refuses a stale one).  `inject_fault` ends a worker process from the host —
the hook the fault-tolerance tests use; nothing here touches a GPU.

Reference: miles/utils/workers/ray_worker_manager.py:56-171 (launch, get_worker_addrs, get_cell_infos, inject_fault,
generation check), :208-310 (`_CellManager`), :312-437 (`_BaseActorManager`), process_supervisor.py:81-152.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field

from ..worker_spec import CommandWorkerSpec, PlannedWorker, PortAllocator, plan
from .provider import CellInfo, WorkerInfo, cell_name, worker_name


@dataclass
class _Worker:
    planned: PlannedWorker
    proc: subprocess.Popen | None = None
    log: str | None = None


@dataclass
class _Cell:
    pool: str
    index: int
    workers: list[_Worker] = field(default_factory=list)
    generation: int = 0
    restarts: int = 0

    @property
    def cell_id(self) -> str:
        return cell_name(self.pool, self.index)

    def alive(self) -> bool:
        return bool(self.workers) and all(w.proc is not None and w.proc.poll() is None for w in self.workers)


class StaleGeneration(RuntimeError):
    pass


class WorkerManager:
    def __init__(self, log_dir: str | None = None, host: str = "127.0.0.1"):
        self.cells: dict[str, _Cell] = {}
        self.log_dir, self.host = log_dir, host
        self.lock = threading.RLock()
        self.ports = PortAllocator(host=host)

    # ---- launch ------------------------------------------------------------------------------------------------
    def launch(self, specs: list, nodes: dict[str, int] | None = None, colocate: bool = False, dry_run: bool = False,
               first_slot: int = 0) -> list[dict]:
        nodes = nodes or {"local": max(1, _gpu_count())}
        described = []
        with self.lock:
            for w in plan(specs, nodes, colocate=colocate, ports=self.ports, master_addr=self.host, first_slot=first_slot):
                cell = self.cells.setdefault(cell_name(w.pool, w.cell), _Cell(w.pool, w.cell))
                cell.workers.append(_Worker(w))
                described.append({"name": worker_name(w.pool, w.cell, w.rank), "cmd": self._command(w), "env": w.env, "ports": w.ports})
            if not dry_run:
                for cell in self.cells.values():
                    for wk in cell.workers:
                        if wk.proc is None:
                            self._start(cell, wk)
        return described

    def _command(self, w: PlannedWorker) -> list[str]:
        if isinstance(w.spec, CommandWorkerSpec):
            return list(w.command)
        port = w.ports.get("rpc") or self.ports.get()
        w.ports["rpc"] = port
        return [sys.executable, "-m", "miles_b200.orchestration.worker_spec", "--serve", w.spec.target, "--port", str(port),
                "--kwargs", repr(w.spec.init_kwargs)]

    def _start(self, cell: _Cell, wk: _Worker):
        w = wk.planned
        env = {**os.environ, **w.env, "MILES_WORKER_NAME": worker_name(w.pool, w.cell, w.rank),
               "MILES_WORKER_GENERATION": str(cell.generation)}
        for k in [k for k, v in env.items() if v == "__inherit__"]:      # a spec may hand a planner-set variable back to the parent's value
            if k in os.environ:
                env[k] = os.environ[k]
            else:
                del env[k]
        out = None
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
            wk.log = os.path.join(self.log_dir, f"{worker_name(w.pool, w.cell, w.rank)}.g{cell.generation}.log")
            out = open(wk.log, "ab")
        wk.proc = subprocess.Popen(self._command(w), env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                                   start_new_session=True)

    # ---- queries -----------------------------------------------------------------------------------------------
    def _info(self, cell: _Cell, wk: _Worker) -> WorkerInfo:
        w = wk.planned
        cls = None if isinstance(w.spec, CommandWorkerSpec) else w.spec.target
        return WorkerInfo(worker_name(w.pool, w.cell, w.rank), w.pool, cell.cell_id, w.rank, cell.generation, self.host,
                          tuple(sorted(w.ports.items())), wk.proc.pid if wk.proc else None, cls)

    def get_cell_infos(self, pools: list[str] | None = None) -> dict[str, CellInfo]:
        with self.lock:
            return {cid: CellInfo(cid, c.pool, c.generation, c.alive(), tuple(self._info(c, w) for w in c.workers))
                    for cid, c in self.cells.items() if pools is None or c.pool in pools}

    def num_cells(self, pool: str) -> int:
        return sum(1 for c in self.cells.values() if c.pool == pool)

    def get_worker(self, name: str, expected_generation: int | None = None) -> WorkerInfo:
        with self.lock:
            for c in self.cells.values():
                for wk in c.workers:
                    info = self._info(c, wk)
                    if info.name == name:
                        if expected_generation is not None and expected_generation != c.generation:
                            raise StaleGeneration(f"{name}: generation {c.generation}, caller expected {expected_generation}")
                        return info
        raise KeyError(name)

    def get_worker_infos(self, cell_id: str) -> list[WorkerInfo]:
        with self.lock:
            c = self.cells[cell_id]
            return [self._info(c, w) for w in c.workers]

    def log_tail(self, name: str, n: int = 20) -> str:
        for c in self.cells.values():
            for wk in c.workers:
                if worker_name(wk.planned.pool, wk.planned.cell, wk.planned.rank) == name and wk.log and os.path.exists(wk.log):
                    return "".join(open(wk.log, errors="replace").readlines()[-n:])
        return ""

    # ---- lifecycle ---------------------------------------------------------------------------------------------
    def _stop_proc(self, p: subprocess.Popen | None, grace: float = 10.0):
        if p is None or p.poll() is not None:
            return
        try:
            os.killpg(p.pid, signal.SIGTERM)          # the worker's own session: the group is exactly what it spawned
        except (ProcessLookupError, PermissionError):
            p.terminate()
        try:
            p.wait(timeout=grace)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(p.pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                p.kill()
            p.wait(timeout=grace)

    def stop_cell(self, cell_id: str):
        with self.lock:
            for wk in self.cells[cell_id].workers:
                self._stop_proc(wk.proc)

    def restart_cell(self, cell_id: str) -> CellInfo:
        with self.lock:
            c = self.cells[cell_id]
            for wk in c.workers:
                self._stop_proc(wk.proc)
            c.generation += 1
            c.restarts += 1
            for wk in c.workers:
                self._start(c, wk)
            return self.get_cell_infos()[cell_id]

    def inject_fault(self, cell_id: str, mode: str = "kill", worker_in_cell_index: int = 0):
        """End (`kill`: SIGKILL, `term`: SIGTERM) or freeze (`stop`: SIGSTOP) one worker process of a cell."""
        sig = {"kill": signal.SIGKILL, "term": signal.SIGTERM, "stop": signal.SIGSTOP}[mode]
        with self.lock:
            p = self.cells[cell_id].workers[worker_in_cell_index].proc
        if p is not None and p.poll() is None:
            os.kill(p.pid, sig)

    def stop_all(self):
        with self.lock:
            for c in self.cells.values():
                for wk in c.workers:
                    self._stop_proc(wk.proc)

    def wait_exit(self, cell_id: str, timeout: float = 10.0) -> bool:
        end = time.monotonic() + timeout
        while time.monotonic() < end:
            if not self.cells[cell_id].alive():
                return True
            time.sleep(0.05)
        return False


def _gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0
