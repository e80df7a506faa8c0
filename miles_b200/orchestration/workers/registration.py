"""Self-registration of workers that this job did not launch.

A REPORTER runs next to some workers (one per node or per deployment), watches the cells it can see through any
provider, and posts a snapshot `{reporter_id, seq, cells}` to the HUB whenever something changed (debounced) and at
least every `interval` seconds as a heartbeat.  The HUB is itself a worker provider: its cells are the union of the
latest snapshot of every reporter that is still posting; a reporter silent for `ttl` seconds is dropped together with
its cells, and a snapshot with an older sequence number than the last one from that reporter is ignored.

Reference: miles/utils/workers/registration/hub.py:28-161 (ingest, stale reporter removal, addressability checks),
reporter.py:28-146 (debounced interval trigger, snapshot), models.py.
"""
from __future__ import annotations

try:  # module level: route signatures are resolved against module globals
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse
except ImportError:  # the HTTP surface is optional
    FastAPI = HTTPException = Request = JSONResponse = None

import asyncio
import json
import time
from dataclasses import asdict

from .provider import BaseWorkerProvider, CellInfo, WorkerInfo


def cell_to_json(c: CellInfo) -> dict:
    d = asdict(c)
    d["workers"] = [asdict(w) for w in c.workers]
    return d


def cell_from_json(d: dict) -> CellInfo:
    ws = tuple(WorkerInfo(**{**w, "ports": tuple(tuple(p) for p in w["ports"])}) for w in d["workers"])
    return CellInfo(d["cell_id"], d["pool"], d["generation"], d["alive"], ws)


class RegistrationHub(BaseWorkerProvider):
    def __init__(self, ttl: float = 30.0, clock=time.monotonic):
        self.ttl, self.clock = ttl, clock
        self.reporters: dict[str, dict] = {}          # id → {seq, seen, cells}

    def ingest(self, snapshot: dict) -> bool:
        rid, seq = snapshot["reporter_id"], int(snapshot.get("seq", 0))
        cells = {c["cell_id"]: cell_from_json(c) for c in snapshot.get("cells", [])}
        for cid, c in cells.items():
            for w in c.workers:
                if not w.host or not w.ports:
                    raise ValueError(f"reporter {rid}: worker {w.name} of cell {cid} has no address")
            owner = next((r for r, st in self.reporters.items() if r != rid and cid in st["cells"]), None)
            if owner is not None:
                raise ValueError(f"cell {cid} is already reported by {owner}")
        st = self.reporters.get(rid)
        if st is not None and seq < st["seq"]:
            return False                                # a delayed older snapshot
        self.reporters[rid] = {"seq": seq, "seen": self.clock(), "cells": cells}
        return True

    def remove_stale(self) -> list[str]:
        now = self.clock()
        gone = [r for r, st in self.reporters.items() if now - st["seen"] > self.ttl]
        for r in gone:
            del self.reporters[r]
        return gone

    async def list_cells(self):
        self.remove_stale()
        out: dict[str, CellInfo] = {}
        for st in self.reporters.values():
            out.update(st["cells"])
        return out

    # ---- HTTP surface ------------------------------------------------------------------------------------------
    def build_app(self):
        app = FastAPI(title="miles_b200 registration hub")

        @app.post("/register")
        async def register(request: Request):
            try:
                accepted = self.ingest(await request.json())
            except (KeyError, ValueError, TypeError) as e:
                raise HTTPException(status_code=422, detail=str(e))
            return {"accepted": accepted, "reporters": len(self.reporters)}

        @app.get("/cells")
        async def cells():
            return {"cells": [cell_to_json(c) for c in (await self.list_cells()).values()]}

        return app

    def serve(self, host="127.0.0.1", port=30200):
        import threading

        import uvicorn

        server = uvicorn.Server(uvicorn.Config(self.build_app(), host=host, port=port, log_level="warning"))
        t = threading.Thread(target=server.run, daemon=True, name=f"registration-hub-{port}")
        t.start()
        while not server.started:
            time.sleep(0.01)
        return server, t


class RegistrationReporter:
    def __init__(self, reporter_id: str, provider: BaseWorkerProvider, post, interval: float = 10.0, debounce: float = 0.2):
        """`post(snapshot_dict)` is an async callable (HTTP POST to the hub's /register, or `hub.ingest` in-process)."""
        self.id, self.provider, self.post = reporter_id, provider, post
        self.interval, self.debounce = interval, debounce
        self.cells: dict[str, CellInfo] = {}
        self.seq = 0
        self.changed = asyncio.Event()
        self.sent = 0

    async def _observe(self, cell_id, info):
        if info is None:
            self.cells.pop(cell_id, None)
        else:
            self.cells[cell_id] = info
        self.changed.set()

    def snapshot(self) -> dict:
        self.seq += 1
        return {"reporter_id": self.id, "seq": self.seq, "cells": [cell_to_json(c) for c in self.cells.values()]}

    async def run(self, watch_interval: float = 1.0):
        stop = await self.provider.watch_cells(self._observe, interval=watch_interval)
        try:
            while True:
                await self.post(self.snapshot())
                self.sent += 1
                self.changed.clear()
                try:
                    await asyncio.wait_for(self.changed.wait(), timeout=self.interval)
                    await asyncio.sleep(self.debounce)       # let a burst of changes settle into one snapshot
                except asyncio.TimeoutError:
                    pass                                     # heartbeat
        finally:
            await stop()


def http_poster(hub_url: str):
    async def post(snapshot: dict):
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=10)) as s:
            async with s.post(hub_url.rstrip("/") + "/register", data=json.dumps(snapshot),
                              headers={"content-type": "application/json"}) as r:
                r.raise_for_status()
                return await r.json()

    return post
