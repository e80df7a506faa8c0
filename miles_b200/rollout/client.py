"""Engine clients used by generate functions.

`InProcEngineClient` drives one or more `Engine` objects living in this process (colocated mode):
requests are queued with a completion callback and a background engine loop (or, in `sync_drive`
mode, the awaiting coroutine itself) steps the engine.  `HttpEngineClient` posts to a router / server
exposing the `/generate` contract (reference client: miles/backends/sglang_utils/sglang_api_client.py:58-460).
"""
from __future__ import annotations

import asyncio
from typing import Any


class InProcEngineClient:
    def __init__(self, engines, tokenizer=None, policy: str = "least_active"):
        self.engines = list(engines) if isinstance(engines, (list, tuple)) else [engines]
        self.tokenizer = tokenizer
        self.policy = policy
        self._active = [0] * len(self.engines)
        self._rr = 0
        cfg = self.engines[0].cfg
        self.num_moe_layers = self.engines[0].model.num_moe_layers if cfg.is_moe else 0
        self.moe_topk = cfg.moe_topk
        self._driver: asyncio.Task | None = None
        self.sync_drive = True   # step engines from the event loop instead of background threads
        self._pending: set = set()

    async def start(self):
        if self.sync_drive:
            if self._driver is None or self._driver.done():
                self._driver = asyncio.ensure_future(self._drive())
        else:
            for e in self.engines:
                e.start_loop()

    async def _drive(self):
        try:
            await self._drive_loop()
        except BaseException as exc:   # surface engine failures to every waiting generate() call
            for fut in list(self._pending):
                if not fut.done():
                    fut.set_exception(RuntimeError(f"engine step failed: {type(exc).__name__}: {exc}"))
            raise

    async def _drive_loop(self):
        idle = 0
        lockstep = any(e.lockstep_group is not None for e in self.engines)
        while True:
            busy = False
            for e in self.engines:
                busy |= e.step()
            if lockstep:
                # every step is a collective: keep stepping until all ranks declared their rollout finished
                if not busy and all(e.global_done for e in self.engines):
                    break
            else:
                idle = 0 if busy else idle + 1
                if idle >= 3:
                    if not self._pending:
                        break
                    # requests are waiting but the engine is paused (a weight update in progress): poll, do not spin
                    await asyncio.sleep(0.001)
            await asyncio.sleep(0)  # let finished requests' awaiters run and new ones enqueue

    async def begin(self):
        for e in self.engines:
            e.begin_rollout()
        await self.start()

    async def finish(self):
        """Declare this rank's rollout complete and wait until every lockstep peer has done the same."""
        for e in self.engines:
            e.finish_rollout()
        if self.sync_drive and self._driver is not None:
            await self._driver

    def _pick(self, routing_key=None) -> int:
        if routing_key is not None and self.policy == "consistent_hashing":
            import zlib
            return zlib.crc32(str(routing_key).encode()) % len(self.engines)
        if self.policy == "round_robin":
            self._rr = (self._rr + 1) % len(self.engines)
            return self._rr
        return min(range(len(self.engines)), key=lambda i: self._active[i])

    async def generate(self, payload: dict, routing_key=None) -> dict:
        i = self._pick(routing_key)
        eng = self.engines[i]
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()

        def on_done(req):
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(req))

        self._active[i] += 1
        self._pending.add(fut)
        try:
            eng.add_request(payload["input_ids"], payload.get("sampling_params"), payload.get("return_logprob", True),
                            payload.get("return_routed_experts", False), on_done=on_done,
                            logprob_start_len=payload.get("logprob_start_len", -1),
                            top_logprobs_num=payload.get("top_logprobs_num", 0))
            await self.start()
            req = await fut
        finally:
            self._active[i] -= 1
            self._pending.discard(fut)
        return req.to_response(eng, raw_routed=True)

    async def abort_all(self):
        for e in self.engines:
            e.abort_request(None)

    async def call_all(self, method: str, *a, **kw) -> list:
        return [getattr(e, method)(*a, **kw) for e in self.engines]


class HttpEngineClient:
    def __init__(self, base_url: str, tokenizer=None, num_moe_layers: int = 0, moe_topk: int = 0, timeout: float = 3600.0,
                 worker_urls: list[str] | None = None):
        self.base_url = base_url.rstrip("/")
        self.worker_urls = worker_urls or []
        self.tokenizer = tokenizer
        self.num_moe_layers, self.moe_topk = num_moe_layers, moe_topk
        self.timeout = timeout
        self._session = None

    async def start(self):
        if self._session is None:
            import aiohttp
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout))

    async def close(self):
        if self._session is not None:
            await self._session.close()
            self._session = None

    async def _post(self, url: str, body: dict | None = None, headers: dict | None = None, retries: int = 3) -> Any:
        await self.start()
        last = None
        for attempt in range(retries):
            try:
                async with self._session.post(url, json=body or {}, headers=headers) as resp:
                    resp.raise_for_status()
                    ctype = resp.headers.get("content-type", "")
                    return await resp.json() if "json" in ctype else await resp.text()
            except Exception as e:  # network hiccup: back off and retry
                last = e
                await asyncio.sleep(0.2 * (attempt + 1))
        raise last

    async def generate(self, payload: dict, routing_key=None) -> dict:
        headers = {"X-SMG-Routing-Key": str(routing_key)} if routing_key is not None else None
        return await self._post(f"{self.base_url}/generate", payload, headers)

    async def abort_all(self):
        targets = self.worker_urls or [self.base_url]
        await asyncio.gather(*[self._post(f"{u}/abort_request", {"abort_all": True}) for u in targets])

    async def begin(self):
        await self.start()

    async def finish(self):
        await self.close()            # the session belongs to the event loop of this rollout; the next one opens its own

    async def call_all(self, endpoint: str, body: dict | None = None) -> list:
        targets = self.worker_urls or [self.base_url]
        return await asyncio.gather(*[self._post(f"{u}/{endpoint.lstrip('/')}", body) for u in targets])
