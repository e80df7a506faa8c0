"""Control API over the job's cells, and the in-job controller loop that heals through it.

    GET   /api/v1/health
    GET   /api/v1/cells                      → {"items": [Cell, …]}
    GET   /api/v1/cells/{name}               → Cell
    PATCH /api/v1/cells/{name}               body {"spec": {"suspend": true|false}}: fence / re-admit a cell
    POST  /api/v1/cells/{name}/inject-fault  body {"mode": "kill"|"term"|"stop"|"raise", "sub_index": 0}

A Cell is described the way a cluster API describes a resource: `metadata` (name, labels: cell type and index), `spec`
(suspend) and `status` (generation + three tri-state conditions: Allocated — it has workers; Healthy — its last probe or
call succeeded; Serving — it takes part in steps).  Errors come back as status objects (`reason`: NotFound, BadRequest,
Conflict).  Two kinds of cells are served: the trainer's replicas (`CellController`) and the rollout servers
(`InferenceController`, with the worker fleet behind it when engines are separate processes).  Fault injection acts on
the HOST only: a worker process is signalled, or the trainer cell's next call raises — nothing here reaches a GPU.

`MiniFTController` is the loop an operator would otherwise run outside the job: poll the API; a cell that is allocated
but unhealthy is suspended, left fenced for a delay that doubles with every consecutive failure, then resumed.

Reference: miles/utils/ft_utils/api_server/server.py:29-203, handles.py:17-111, models.py:13-97,
mini_ft_controller.py:25-230.
"""
from __future__ import annotations

try:  # module level: route signatures are resolved against module globals
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse
except ImportError:  # the HTTP surface is optional
    FastAPI = HTTPException = Request = JSONResponse = None

import threading
import time
from typing import Any

TRUE, FALSE, UNKNOWN = "True", "False", "Unknown"


def condition(kind: str, status: str, reason: str | None = None) -> dict:
    return {"type": kind, "status": status, **({"reason": reason} if reason else {})}


def make_cell(name: str, cell_type: str, index: int, *, suspend: bool, generation: int, allocated: str, healthy: str,
              serving: str, reason: str | None = None) -> dict:
    phase = "Suspended" if suspend else ("Running" if healthy == TRUE else ("Failed" if healthy == FALSE else "Pending"))
    return {"apiVersion": "miles/v1", "kind": "Cell",
            "metadata": {"name": name, "labels": {"cell-type": cell_type, "cell-index": str(index)}},
            "spec": {"suspend": suspend},
            "status": {"phase": phase, "generation": generation,
                       "conditions": [condition("Allocated", allocated), condition("Healthy", healthy, reason),
                                      condition("Serving", serving)]}}


class ApiError(Exception):
    def __init__(self, code: int, reason: str, message: str):
        super().__init__(message)
        self.code, self.reason, self.message = code, reason, message

    def body(self) -> dict:
        return {"kind": "Status", "apiVersion": "v1", "status": "Failure", "reason": self.reason, "code": self.code,
                "message": self.message}


class TrainerCellHandler:
    """Cells of a `ft.controller.CellController` (or one pseudo-cell for a trainer that runs without it)."""

    cell_type = "trainer"

    def __init__(self, trainer, make_workers=None):
        self.trainer = trainer
        self.make_workers = make_workers              # cell id → fresh worker handles, used by resume
        self.suspended: set[int] = set()

    def _cells(self):
        ctl = getattr(self.trainer, "cells", None)
        return ctl.cells if ctl is not None else {}

    def names(self) -> list[str]:
        return [f"trainer-{i}" for i in sorted(self._cells())] or ["trainer-0"]

    def get(self, name: str) -> dict:
        from .controller import CellState

        i = int(name.rsplit("-", 1)[1])
        cells = self._cells()
        if not cells:
            return make_cell(name, self.cell_type, 0, suspend=False, generation=0, allocated=TRUE, healthy=TRUE, serving=TRUE)
        c = cells[i]
        ok = c.state in (CellState.ALIVE, CellState.UNINITIALIZED)
        return make_cell(name, self.cell_type, i, suspend=i in self.suspended, generation=c.generation,
                         allocated=TRUE if c.workers else FALSE, healthy=TRUE if ok else FALSE, serving=TRUE if ok else FALSE,
                         reason=None if ok else repr(c.error))

    def suspend(self, name: str):
        i = int(name.rsplit("-", 1)[1])
        c = self._cells().get(i)
        if c is None:
            raise ApiError(409, "Conflict", "this trainer runs without fault tolerance: nothing to fence")
        self.suspended.add(i)
        c.mark_errored(RuntimeError("suspended through the API"))
        self.trainer.cells._publish()

    def resume(self, name: str):
        i = int(name.rsplit("-", 1)[1])
        c = self._cells().get(i)
        if c is None:
            raise ApiError(409, "Conflict", "this trainer runs without fault tolerance")
        self.suspended.discard(i)
        workers = self.make_workers(i) if self.make_workers else c.workers
        self.trainer.cells.heal(i, workers)

    def inject_fault(self, name: str, mode: str, sub_index: int):
        from ..testing import fault_injector

        if mode != "raise":
            raise ApiError(400, "BadRequest", "a trainer cell of this process takes mode 'raise' (its next call raises)")
        fault_injector.arm("train", RuntimeError(f"fault injected into {name}"))


class RolloutCellHandler:
    cell_type = "rollout"

    def __init__(self, controller, fleet=None):
        self.ctl, self.fleet = controller, fleet
        self.suspended: set[int] = set()

    def names(self) -> list[str]:
        return [f"rollout-{i}" for i in range(len(self.ctl.cells))]

    def _fleet_cell(self, i: int):
        if self.fleet is None:
            return None, None
        eng = self.ctl.cells[i].engine
        cid = next((k for k, e in self.fleet.engines.items() if e is eng), None)
        return cid, (self.fleet.manager.get_cell_infos().get(cid) if cid and self.fleet.manager else None)

    def get(self, name: str) -> dict:
        i = int(name.rsplit("-", 1)[1])
        c = self.ctl.cells[i]
        _, info = self._fleet_cell(i)
        allocated = TRUE if (info is None or info.alive) else FALSE
        healthy = FALSE if c.state == "unhealthy" or allocated == FALSE else TRUE
        serving = TRUE if c.state in ("alive", "stale") and healthy == TRUE else FALSE
        return make_cell(name, self.cell_type, i, suspend=i in self.suspended, generation=info.generation if info else 0,
                         allocated=allocated, healthy=healthy, serving=serving, reason=None if healthy == TRUE else c.state)

    def suspend(self, name: str):
        i = int(name.rsplit("-", 1)[1])
        c = self.ctl.cells[i]
        self.suspended.add(i)
        try:
            c.engine.pause_generation("abort")
        except Exception:
            pass                                      # an engine that no longer answers is fenced all the same
        c.state = "unhealthy"

    def resume(self, name: str):
        i = int(name.rsplit("-", 1)[1])
        c = self.ctl.cells[i]
        self.suspended.discard(i)
        c.engine.continue_generation()
        behind = hasattr(c.engine, "get_weight_version") and c.engine.get_weight_version() != self.ctl.weight_version
        c.state = "stale" if behind else "alive"      # a stale engine is re-synced by the next weight update

    def inject_fault(self, name: str, mode: str, sub_index: int):
        i = int(name.rsplit("-", 1)[1])
        cid, _ = self._fleet_cell(i)
        if cid is None or self.fleet.manager is None:
            raise ApiError(400, "BadRequest", "this rollout cell is not a process launched by the job")
        if mode not in ("kill", "term", "stop"):
            raise ApiError(400, "BadRequest", f"unknown mode {mode!r}")
        self.fleet.manager.inject_fault(cid, mode=mode, worker_in_cell_index=sub_index)


class CellRegistry:
    def __init__(self, handlers: list):
        self.handlers = handlers

    def resolve(self, name: str):
        for h in self.handlers:
            if name in h.names():
                return h
        raise ApiError(404, "NotFound", f"cell {name!r} not found")

    def list(self) -> list[dict]:
        return [h.get(n) for h in self.handlers for n in h.names()]


def create_app(registry: CellRegistry):
    app = FastAPI(title="miles_b200 cell API")

    @app.exception_handler(ApiError)
    async def _err(request: Request, exc: ApiError):
        return JSONResponse(status_code=exc.code, content=exc.body())

    @app.get("/api/v1/health")
    async def health():
        return {"status": "ok"}

    @app.get("/api/v1/cells")
    async def cells():
        return {"apiVersion": "miles/v1", "kind": "CellList", "items": registry.list()}

    @app.get("/api/v1/cells/{name}")
    async def cell(name: str):
        return registry.resolve(name).get(name)

    @app.patch("/api/v1/cells/{name}")
    async def patch(name: str, request: Request):
        body = await request.json()
        spec = body.get("spec") if isinstance(body, dict) else None
        if not isinstance(spec, dict) or not isinstance(spec.get("suspend"), bool) or set(spec) != {"suspend"}:
            raise ApiError(400, "BadRequest", 'the patch must be {"spec": {"suspend": true|false}}')
        h = registry.resolve(name)
        current = h.get(name)["spec"]["suspend"]
        if spec["suspend"] != current:
            (h.suspend if spec["suspend"] else h.resume)(name)
        return h.get(name)

    @app.post("/api/v1/cells/{name}/inject-fault")
    async def inject(name: str, request: Request):
        body = await request.json()
        registry.resolve(name).inject_fault(name, str(body.get("mode", "kill")), int(body.get("sub_index", 0)))
        return {"status": "ok"}

    return app


def start_api_server(args, trainer=None, rollout=None, host: str | None = None, port: int | None = None):
    """Serve the API in a background thread when `--api-server-port` is set; returns (server, thread, registry) or None."""
    port = port if port is not None else getattr(args, "api_server_port", None)
    if not port:
        return None
    import uvicorn

    handlers: list[Any] = []
    if trainer is not None:
        handlers.append(TrainerCellHandler(trainer))
    if rollout is not None and getattr(rollout, "controller", None) is not None:
        handlers.append(RolloutCellHandler(rollout.controller, getattr(rollout, "fleet", None)))
    registry = CellRegistry(handlers)
    server = uvicorn.Server(uvicorn.Config(create_app(registry), host=host or getattr(args, "api_server_host", None) or "127.0.0.1",
                                           port=int(port), log_level="warning"))
    t = threading.Thread(target=server.run, daemon=True, name=f"cell-api-{port}")
    t.start()
    while not server.started:
        time.sleep(0.01)
    return server, t, registry


# ---- the controller loop ------------------------------------------------------------------------------------------

class MiniFTController:
    def __init__(self, get_cells, patch_suspend, poll_interval: float = 10.0, resume_delay: float = 10.0,
                 max_delay: float = 600.0, clock=time.monotonic, sleep=time.sleep):
        self.get_cells, self.patch_suspend = get_cells, patch_suspend
        self.poll_interval, self.resume_delay, self.max_delay = poll_interval, resume_delay, max_delay
        self.clock, self.sleep = clock, sleep
        self.failures: dict[str, int] = {}
        self.resume_at: dict[str, float] = {}
        self.log: list[tuple] = []
        self._stop = threading.Event()

    @staticmethod
    def _cond(cell: dict, kind: str) -> str:
        return next((c["status"] for c in cell["status"]["conditions"] if c["type"] == kind), UNKNOWN)

    def poll_and_heal(self):
        now = self.clock()
        for cell in self.get_cells():
            name = cell["metadata"]["name"]
            suspended = cell["spec"]["suspend"]
            if name in self.resume_at:
                if now >= self.resume_at[name]:
                    del self.resume_at[name]
                    self.patch_suspend(name, False)
                    self.log.append(("resumed", name))
                continue
            if suspended:
                continue                                   # fenced by someone else: not ours to resume
            if self._cond(cell, "Healthy") == FALSE:
                n = self.failures[name] = self.failures.get(name, 0) + 1
                delay = min(self.max_delay, self.resume_delay * (2 ** (n - 1)))
                self.patch_suspend(name, True)
                self.resume_at[name] = now + delay
                self.log.append(("suspended", name, delay))
            elif self._cond(cell, "Healthy") == TRUE and self._cond(cell, "Serving") == TRUE:
                self.failures.pop(name, None)

    def run(self):
        while not self._stop.is_set():
            try:
                self.poll_and_heal()
            except Exception as e:  # the API may be briefly away; the next pass looks again
                self.log.append(("error", repr(e)))
            self._stop.wait(self.poll_interval)

    def request_stop(self):
        self._stop.set()


def http_cell_client(base_url: str):
    import requests

    base = base_url.rstrip("/")

    def get_cells():
        r = requests.get(f"{base}/api/v1/cells", timeout=10)
        r.raise_for_status()
        return r.json()["items"]

    def patch_suspend(name: str, suspend: bool):
        r = requests.patch(f"{base}/api/v1/cells/{name}", json={"spec": {"suspend": suspend}}, timeout=60)
        r.raise_for_status()
        return r.json()

    return get_cells, patch_suspend


def maybe_start_mini_ft_controller(args):
    """`--mini-ft-controller-enable`: run the loop in a daemon thread against this job's own API server."""
    if not getattr(args, "mini_ft_controller_enable", False):
        return None
    port = getattr(args, "api_server_port", None)
    assert port, "--mini-ft-controller-enable needs --api-server-port"
    host = getattr(args, "api_server_host", None) or "127.0.0.1"
    get_cells, patch = http_cell_client(f"http://{host}:{port}")
    ctl = MiniFTController(get_cells, patch, poll_interval=float(getattr(args, "mini_ft_controller_poll_interval", 10.0) or 10.0),
                           resume_delay=float(getattr(args, "mini_ft_controller_resume_delay", 10.0) or 10.0))
    threading.Thread(target=ctl.run, daemon=True, name="mini-ft-controller").start()
    return ctl
