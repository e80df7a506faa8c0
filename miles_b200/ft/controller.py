"""Cells, health checking and a small fault-tolerance controller (host side only).

Reference pieces: `TrainerCell` state machine Uninitialized → Alive → Errored with kill-on-failure
(miles/ray/train/cell.py:29-309), `TrainerController` fan-out with ≤30 retry attempts and healing by refreshing cells
(miles/ray/train/group.py:52-685), the rollout health checker that quarantines engines after consecutive failed
probes, the mini FT controller and the K8s-style cell API (miles/utils/ft_utils/*).

Everything here observes and reacts on the host: heartbeats in a key-value store, HTTP health probes, exceptions
raised by worker calls.  Nothing in this module makes a GPU fault, trap or hang — failures are injected with
`miles_b200.testing.fault_injector` (a rank that raises, exits between steps or drops a message).
"""
from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable


class CellState(enum.Enum):
    UNINITIALIZED = "uninitialized"
    ALIVE = "alive"
    ERRORED = "errored"
    STOPPED = "stopped"


@dataclass
class Cell:
    """One replica: a set of worker handles driven together.  `workers` expose the trainer API as callables
    (`init`, `train`, `update_weights`, `save_model`, …) and a `kill()` used to fence a failed replica."""

    cell_id: int
    workers: list[Any]
    state: CellState = CellState.UNINITIALIZED
    error: BaseException | None = None
    generation: int = 0

    def execute(self, method: str, *args, **kwargs) -> list:
        if self.state not in (CellState.ALIVE, CellState.UNINITIALIZED):
            raise RuntimeError(f"cell {self.cell_id} is {self.state.value}")
        try:
            out = [getattr(w, method)(*args, **kwargs) for w in self.workers]
            if method == "init":
                self.state = CellState.ALIVE
            return out
        except BaseException as e:
            self.mark_errored(e)
            raise

    def mark_errored(self, error: BaseException | None = None):
        self.state, self.error = CellState.ERRORED, error
        for w in self.workers:                  # fence: a half-dead replica must not rejoin a collective
            kill = getattr(w, "kill", None)
            if kill is not None:
                try:
                    kill()
                except Exception:
                    pass

    def replace_workers(self, workers: list[Any]):
        self.workers, self.state, self.error = workers, CellState.UNINITIALIZED, None
        self.generation += 1


class CellController:
    """Fan a call out to every live cell; a failing cell is fenced, the membership shrinks, the call is retried on
    the quorum (at most `max_attempts` times); `heal()` brings replacement workers in and copies state from a donor."""

    def __init__(self, cells: list[Cell], *, min_quorum: int = 1, max_attempts: int = 30,
                 on_membership: Callable[[list[int]], None] | None = None):
        self.cells, self.min_quorum, self.max_attempts = {c.cell_id: c for c in cells}, min_quorum, max_attempts
        self.on_membership = on_membership
        self.epoch = 0
        self.log: list[tuple[str, Any]] = []

    def alive(self) -> list[Cell]:
        return [c for c in self.cells.values() if c.state in (CellState.ALIVE, CellState.UNINITIALIZED)]

    def _publish(self):
        self.epoch += 1
        ids = sorted(c.cell_id for c in self.alive())
        self.log.append(("membership", (self.epoch, ids)))
        if self.on_membership is not None:
            self.on_membership(ids)

    def execute(self, method: str, *args, **kwargs) -> dict[int, list]:
        for attempt in range(self.max_attempts):
            live = self.alive()
            if len(live) < self.min_quorum:
                raise RuntimeError(f"only {len(live)} live cells, quorum is {self.min_quorum}")
            results, failed = {}, []
            for c in live:
                try:
                    results[c.cell_id] = c.execute(method, *args, **kwargs)
                except BaseException as e:
                    failed.append(c.cell_id)
                    self.log.append(("cell_failed", (c.cell_id, method, repr(e))))
            if not failed:
                return results
            self._publish()                    # survivors rebuild their cross-cell group, then the step is retried
        raise RuntimeError(f"{method} did not succeed in {self.max_attempts} attempts")

    def heal(self, cell_id: int, new_workers: list[Any], transfer: Callable[[Cell, Cell], None] | None = None):
        """Re-admit a cell with fresh workers; `transfer(donor, healed)` copies model/optimizer state."""
        cell = self.cells[cell_id]
        cell.replace_workers(new_workers)
        cell.execute("init")
        donors = [c for c in self.alive() if c.cell_id != cell_id and c.state == CellState.ALIVE]
        if transfer is not None and donors:
            transfer(donors[0], cell)
        self.log.append(("healed", cell_id))
        self._publish()


# ---- health ----------------------------------------------------------------------------------------------------

class HeartbeatMonitor:
    """Workers call `beat()`; the monitor reports ids whose last beat is older than `timeout_s`.  Backed by any store
    with `set(key, value)` / `get(key)` (a `dist.TCPStore`, or a dict wrapper in tests)."""

    def __init__(self, store, timeout_s: float = 30.0, prefix: str = "hb", clock: Callable[[], float] = time.time):
        self.store, self.timeout_s, self.prefix, self.clock = store, timeout_s, prefix, clock
        self.known: set[str] = set()

    def beat(self, worker_id: str):
        self.store.set(f"{self.prefix}/{worker_id}", str(self.clock()))
        self.known.add(worker_id)

    def watch(self, worker_id: str):
        self.known.add(worker_id)

    def dead(self) -> list[str]:
        now, out = self.clock(), []
        for w in sorted(self.known):
            try:
                raw = self.store.get(f"{self.prefix}/{w}")
                last = float(raw.decode() if isinstance(raw, bytes) else raw)
            except Exception:
                last = float("-inf")
            if now - last > self.timeout_s:
                out.append(w)
        return out


class EngineHealthChecker:
    """Probe rollout engines (`probe(engine) -> bool`, e.g. GET /health_generate); after `threshold` consecutive
    failures an engine is quarantined and `on_unhealthy(engine)` fires; a later good probe re-admits it."""

    def __init__(self, engines: list[Any], probe: Callable[[Any], bool], threshold: int = 3,
                 on_unhealthy: Callable[[Any], None] | None = None, on_recovered: Callable[[Any], None] | None = None):
        self.engines, self.probe, self.threshold = list(engines), probe, threshold
        self.on_unhealthy, self.on_recovered = on_unhealthy, on_recovered
        self.failures = {id(e): 0 for e in self.engines}
        self.quarantined: set[int] = set()
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()

    def check_once(self):
        for e in self.engines:
            try:
                ok = bool(self.probe(e))
            except Exception:
                ok = False
            k = id(e)
            if ok:
                self.failures[k] = 0
                if k in self.quarantined:
                    self.quarantined.discard(k)
                    if self.on_recovered:
                        self.on_recovered(e)
            else:
                self.failures[k] += 1
                if self.failures[k] >= self.threshold and k not in self.quarantined:
                    self.quarantined.add(k)
                    if self.on_unhealthy:
                        self.on_unhealthy(e)

    def healthy(self) -> list[Any]:
        return [e for e in self.engines if id(e) not in self.quarantined]

    def start(self, interval_s: float = 10.0):
        def loop():
            while not self._stop.wait(interval_s):
                self.check_once()

        self._thread = threading.Thread(target=loop, daemon=True, name="engine-health")
        self._thread.start()

    def stop(self):
        self._stop.set()


@dataclass
class MiniFTController:
    """Ties the pieces together for one job: heartbeat monitor → fence dead cells → publish membership → heal when a
    replacement registers.  `tick()` is one reconcile pass (call it from a loop or a test)."""

    cells: CellController
    monitor: HeartbeatMonitor
    worker_to_cell: dict[str, int] = field(default_factory=dict)
    pending_replacements: dict[int, list[Any]] = field(default_factory=dict)
    transfer: Callable[[Cell, Cell], None] | None = None

    def register_replacement(self, cell_id: int, workers: list[Any]):
        self.pending_replacements[cell_id] = workers

    def tick(self) -> dict:
        fenced, healed = [], []
        for w in self.monitor.dead():
            cid = self.worker_to_cell.get(w)
            cell = self.cells.cells.get(cid) if cid is not None else None
            if cell is not None and cell.state in (CellState.ALIVE, CellState.UNINITIALIZED):
                cell.mark_errored(TimeoutError(f"worker {w} missed its heartbeat"))
                fenced.append(cid)
        if fenced:
            self.cells._publish()
        for cid, workers in list(self.pending_replacements.items()):
            if self.cells.cells[cid].state == CellState.ERRORED:
                self.cells.heal(cid, workers, self.transfer)
                healed.append(cid)
                del self.pending_replacements[cid]
        return {"fenced": fenced, "healed": healed, "alive": sorted(c.cell_id for c in self.cells.alive())}
