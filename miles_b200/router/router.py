"""Request router in front of the rollout engines.

HTTP surface of the reference's router (miles/router/router.py:36-254; production deployments use the Rust
`sgl-model-gateway`): `POST /generate` (and any other path) proxied to a worker chosen by policy, `POST /add_worker`,
`POST /remove_worker`, `GET /list_workers`, `GET /workers`, `GET /health`, `GET /metrics`; background health checks
quarantine workers after consecutive failures and re-admit them when they answer again.  Worker choice
(least-active-requests, round robin, consistent hashing on `X-SMG-Routing-Key`, random) runs in the native runtime
(`miles_b200/native/csrc/runtime.cpp`) when it is built, else in the python fallback below.

    python -m miles_b200.router.router --port 30100 --workers http://127.0.0.1:30000 http://127.0.0.1:30001
"""
from __future__ import annotations

import argparse
import asyncio
import itertools
import random
import time
import zlib

from fastapi import FastAPI, Request, Response   # module level: postponed annotations are resolved in module scope


class _PyCore:
    def __init__(self):
        self.active: list[int] = []
        self.healthy: list[bool] = []
        self.rr = itertools.count()

    def add_worker(self) -> int:
        self.active.append(0)
        self.healthy.append(True)
        return len(self.active) - 1

    def set_health(self, w, ok):
        self.healthy[w] = bool(ok)

    def pick(self, policy="least_active", key=None) -> int:
        ok = [i for i, h in enumerate(self.healthy) if h]
        if not ok:
            return -1
        if policy == "round_robin":
            w = ok[next(self.rr) % len(ok)]
        elif policy == "consistent_hashing" and key:
            w = ok[zlib.crc32(key.encode()) % len(ok)]
        elif policy == "random":
            w = random.choice(ok)
        else:
            w = min(ok, key=lambda i: self.active[i])
        self.active[w] += 1
        return w

    def done(self, w):
        if 0 <= w < len(self.active) and self.active[w] > 0:
            self.active[w] -= 1

    def active_of(self, w):
        return self.active[w]


def _make_core():
    try:
        from ..native import runtime as rt

        if rt.available():
            core = rt.NativeRouterCore(0)
            core.active_of = core.active
            return core
    except Exception:
        pass
    return _PyCore()


class Router:
    def __init__(self, policy: str = "least_active", health_interval: float = 10.0, health_timeout: float = 5.0,
                 failure_threshold: int = 3):
        self.policy = policy
        self.core = _make_core()
        self.urls: list[str | None] = []
        self.failures: list[int] = []
        self.health_interval, self.health_timeout, self.failure_threshold = health_interval, health_timeout, failure_threshold
        self.stats = {"requests": 0, "errors": 0}
        self._session = None
        self._health_task = None

    # ---- worker set ----------------------------------------------------------------------------
    def add_worker(self, url: str) -> int:
        url = url.rstrip("/")
        if url in self.urls:
            i = self.urls.index(url)
            self.core.set_health(i, True)
            self.failures[i] = 0
            return i
        i = self.core.add_worker()
        self.urls.append(url)
        self.failures.append(0)
        return i

    def remove_worker(self, url: str) -> bool:
        url = url.rstrip("/")
        if url not in self.urls:
            return False
        i = self.urls.index(url)
        self.core.set_health(i, False)
        self.urls[i] = None
        return True

    def list_workers(self) -> list[str]:
        return [u for u in self.urls if u]

    # ---- proxy -----------------------------------------------------------------------------------
    async def session(self):
        if self._session is None:
            import aiohttp

            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))
        return self._session

    async def forward(self, path: str, method: str, body: bytes, headers: dict) -> tuple[int, bytes, str]:
        key = headers.get("x-smg-routing-key") or headers.get("X-SMG-Routing-Key")
        w = self.core.pick(self.policy, key)
        if w < 0:
            return 503, b'{"error": "no healthy worker"}', "application/json"
        self.stats["requests"] += 1
        try:
            s = await self.session()
            async with s.request(method, f"{self.urls[w]}/{path.lstrip('/')}", data=body or None,
                                 headers={"content-type": headers.get("content-type", "application/json")}) as resp:
                data = await resp.read()
                return resp.status, data, resp.headers.get("content-type", "application/json")
        except Exception as e:
            self.stats["errors"] += 1
            self._note_failure(w)
            return 502, f'{{"error": "worker {self.urls[w]} failed: {type(e).__name__}"}}'.encode(), "application/json"
        finally:
            self.core.done(w)

    def _note_failure(self, w: int):
        self.failures[w] += 1
        if self.failures[w] >= self.failure_threshold:
            self.core.set_health(w, False)

    async def health_loop(self):
        while True:
            await asyncio.sleep(self.health_interval)
            await self.check_health_once()

    async def check_health_once(self):
        import aiohttp

        s = await self.session()
        for i, url in enumerate(self.urls):
            if not url:
                continue
            try:
                async with s.get(f"{url}/health", timeout=aiohttp.ClientTimeout(total=self.health_timeout)) as r:
                    ok = r.status == 200
            except Exception:
                ok = False
            if ok:
                self.failures[i] = 0
                self.core.set_health(i, True)
            else:
                self._note_failure(i)


def build_app(router: Router):
    app = FastAPI(title="miles_b200 router")

    @app.on_event("startup")
    async def _start():
        router._health_task = asyncio.ensure_future(router.health_loop())

    @app.post("/add_worker")
    async def add_worker(request: Request):
        url = request.query_params.get("url") or (await request.json()).get("url")
        return {"worker_id": router.add_worker(url), "workers": router.list_workers()}

    @app.post("/remove_worker")
    async def remove_worker(request: Request):
        url = request.query_params.get("url") or (await request.json()).get("url")
        return {"removed": router.remove_worker(url), "workers": router.list_workers()}

    @app.get("/list_workers")
    async def list_workers():
        return {"urls": router.list_workers()}

    @app.get("/workers")
    async def workers():
        return {"workers": [{"url": u, "active": router.core.active_of(i), "failures": router.failures[i]}
                            for i, u in enumerate(router.urls) if u]}

    @app.get("/health")
    async def health():
        return {"status": "ok", "workers": len(router.list_workers())}

    @app.get("/metrics")
    async def metrics():
        body = "".join(f"router_{k}_total {v}\n" for k, v in router.stats.items())
        return Response(body, media_type="text/plain")

    @app.api_route("/{path:path}", methods=["GET", "POST"])
    async def proxy(path: str, request: Request):
        status, data, ctype = await router.forward(path, request.method, await request.body(), dict(request.headers))
        return Response(data, status_code=status, media_type=ctype)

    return app


def serve(router: Router, host="127.0.0.1", port=30100, in_thread=False):
    import threading

    import uvicorn

    server = uvicorn.Server(uvicorn.Config(build_app(router), host=host, port=port, log_level="warning"))
    if in_thread:
        t = threading.Thread(target=server.run, daemon=True, name=f"router-{port}")
        t.start()
        while not server.started:
            time.sleep(0.01)
        return server, t
    server.run()


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30100)
    p.add_argument("--policy", default="least_active", choices=["least_active", "round_robin", "consistent_hashing", "random"])
    p.add_argument("--workers", nargs="*", default=[])
    a = p.parse_args()
    r = Router(a.policy)
    for w in a.workers:
        r.add_worker(w)
    serve(r, a.host, a.port)


if __name__ == "__main__":
    main()
