"""Prefill / decode disaggregation: prompts run on prefill engines, generation continues on decode engines.

The serving stack the reference drives can split an engine fleet into prefill and decode workers (its `--sglang-config`
worker types `prefill` / `decode` behind a router in PD mode, miles/backends/sglang_utils/sglang_config.py): long prompts
then never stall the decode batches of other requests.  Here the hand-over is explicit and small: a prefill engine runs
the prompt with `keep_kv`, samples the first token and keeps the request's cache blocks; `Engine.export_kv` gathers
them into one tensor [layers, 2, tokens, kv heads, head dim]; the decode engine allocates blocks, stores the tensor
(`Engine.add_prefilled`) and decodes from the first token on; the prefill engine then releases its blocks.  Engines may sit on
different GPUs of the box (the tensor crosses NVLink once, as one copy) or in other processes (`engine/server.py`:
`/prefill` → `/generate_prefilled` with the tensor as a CUDA-IPC bucket, `/release_kv`).

`PDClient` has the interface of the in-process engine client, so a rollout function runs on a PD pair unchanged.
"""
from __future__ import annotations

import asyncio

from ..rollout.client import InProcEngineClient


class PDClient(InProcEngineClient):
    """In-process PD serving: `prefill` and `decode` are lists of engines (weights kept in sync by the caller: both lists are
    in `self.engines`, so weight updates and cache flushes through `call_all` reach every engine)."""

    def __init__(self, prefill: list, decode: list, tokenizer=None):
        super().__init__(list(prefill) + list(decode), tokenizer=tokenizer)
        self.prefill, self.decode = list(prefill), list(decode)
        self._p_active = [0] * len(self.prefill)
        self._d_active = [0] * len(self.decode)
        self.stats = {"handed_over_tokens": 0, "requests": 0}

    async def _await_request(self, add):
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()

        def on_done(req):
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(req))

        self._pending.add(fut)
        try:
            add(on_done)
            await self.start()
            return await fut
        finally:
            self._pending.discard(fut)

    async def generate(self, payload: dict, routing_key=None) -> dict:
        sp = dict(payload.get("sampling_params") or {})
        want_routed = payload.get("return_routed_experts", False)
        pi = min(range(len(self.prefill)), key=lambda i: self._p_active[i])
        P = self.prefill[pi]
        self._p_active[pi] += 1
        try:
            first = await self._await_request(lambda cb: P.add_request(
                payload["input_ids"], {**sp, "max_new_tokens": 1}, payload.get("return_logprob", True), want_routed, on_done=cb,
                logprob_start_len=payload.get("logprob_start_len", -1), top_logprobs_num=payload.get("top_logprobs_num", 0),
                keep_kv=True))
        finally:
            self._p_active[pi] -= 1
        head = first.to_response(P, raw_routed=True)
        if first.rid not in P.held_kv or int(sp.get("max_new_tokens", 128)) <= 1 or first.finish_reason.get("type") == "stop":
            P.release_kv(first.rid)                       # nothing to continue: the prefill engine's reply is the answer
            return head
        di = min(range(len(self.decode)), key=lambda i: self._d_active[i])
        D = self.decode[di]
        self._d_active[di] += 1
        try:
            kv = P.export_kv(first.rid)
            n = len(first.input_ids)
            routed = head["meta_info"].get("routed_experts")
            rest = await self._await_request(lambda cb: D.add_prefilled(
                first.input_ids, first.output_ids[0], first.output_logprobs[0], kv, sp, payload.get("return_logprob", True),
                want_routed, routed=routed, on_done=cb, seed=first.seed))
            self.stats["handed_over_tokens"] += n
            self.stats["requests"] += 1
        finally:
            P.release_kv(first.rid)
            self._d_active[di] -= 1
        out = rest.to_response(D, raw_routed=True)
        for k in ("input_token_logprobs", "input_top_logprobs"):          # prompt scores come from the engine that ran the prompt
            if k in head["meta_info"]:
                out["meta_info"][k] = head["meta_info"][k]
        out["meta_info"]["prefill_engine"], out["meta_info"]["decode_engine"] = pi, di
        return out


class PDHttpClient:
    """The same over HTTP: `prefill_urls` / `decode_urls` are engine servers (`engine/server.py`); the KV travels as a CUDA-IPC
    handle between processes of one box (bytes from CPU engines)."""

    def __init__(self, prefill_urls: list[str], decode_urls: list[str], tokenizer=None, num_moe_layers: int = 0, moe_topk: int = 0,
                 timeout: float = 3600.0):
        self.prefill_urls, self.decode_urls = [u.rstrip("/") for u in prefill_urls], [u.rstrip("/") for u in decode_urls]
        self.tokenizer, self.num_moe_layers, self.moe_topk, self.timeout = tokenizer, num_moe_layers, moe_topk, timeout
        self._session = None
        self._rr = [0, 0]
        self.stats = {"requests": 0}

    async def _post(self, url: str, body: dict) -> dict:
        import aiohttp

        if self._session is None:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout))
        async with self._session.post(url, json=body) as r:
            r.raise_for_status()
            return await r.json()

    async def start(self):
        pass

    async def begin(self):
        pass

    async def abort_all(self):
        import asyncio

        await asyncio.gather(*[self._post(f"{u}/abort_request", {"abort_all": True}) for u in self.prefill_urls + self.decode_urls])

    async def call_all(self, endpoint: str, body: dict | None = None) -> list:
        import asyncio

        return await asyncio.gather(*[self._post(f"{u}/{endpoint.lstrip('/')}", body) for u in self.prefill_urls + self.decode_urls])

    async def finish(self):
        if self._session is not None:
            await self._session.close()
            self._session = None

    async def generate(self, payload: dict, routing_key=None) -> dict:
        self._rr[0] = (self._rr[0] + 1) % len(self.prefill_urls)
        self._rr[1] = (self._rr[1] + 1) % len(self.decode_urls)
        P, D = self.prefill_urls[self._rr[0]], self.decode_urls[self._rr[1]]
        head = await self._post(f"{P}/prefill", payload)
        rid = head["meta_info"]["id"]
        if "kv" not in head:
            return head
        try:
            sp = dict(payload.get("sampling_params") or {})
            if int(sp.get("max_new_tokens", 128)) <= 1 or head["meta_info"]["finish_reason"].get("type") == "stop":
                head.pop("kv", None)
                return head
            lp, tok = head["meta_info"]["output_token_logprobs"][0][:2] if head["meta_info"].get("output_token_logprobs") \
                else (0.0, head["output_ids"][0])
            out = await self._post(f"{D}/generate_prefilled", {
                "input_ids": payload["input_ids"], "first_token": tok, "first_logprob": lp, "kv": head["kv"], "sampling_params": sp,
                "return_logprob": payload.get("return_logprob", True), "return_routed_experts": payload.get("return_routed_experts", False),
                "routed_experts": head["meta_info"].get("routed_experts"), "seed": head.get("seed")})
            for k in ("input_token_logprobs", "input_top_logprobs"):
                if k in head["meta_info"]:
                    out["meta_info"][k] = head["meta_info"][k]
            self.stats["requests"] += 1
            return out
        finally:
            await self._post(f"{P}/release_kv", {"rid": rid})


def _bench_handover():
    """`python -m miles_b200.engine.pd --tokens 2048`: device time of the KV hand-over between two engines of one GPU (or of
    the first and the last GPU of the box) for a prompt of that many tokens — gather on the prefill side, copy, scatter on the
    decode side — at the Qwen3-30B-A3B cache shape (48 layers, 4 KV heads of 128)."""
    import argparse
    import json

    import torch

    from ..models.config import get_config
    from .engine import Engine

    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--layers", type=int, default=48)
    p.add_argument("--iters", type=int, default=10)
    a = p.parse_args()
    cfg = get_config("qwen3-30B-A3B").with_(num_experts=8, num_layers=a.layers, moe_ffn_hidden_size=128, hidden_size=512)
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", torch.cuda.device_count() - 1)
    blocks = (a.tokens + 63) // 64 + 2
    P = Engine(cfg, device=d0, dtype=torch.bfloat16, num_blocks=2 * blocks, max_running_requests=4, max_context_len=a.tokens + 64, seed=0)
    D = Engine(cfg, device=d1, dtype=torch.bfloat16, num_blocks=2 * blocks, max_running_requests=4, max_context_len=a.tokens + 64, seed=0)
    for kc, vc in P.kv.layers.values():
        kc.normal_()
        vc.normal_()
    ids = list(range(3, 3 + a.tokens))
    times = []
    for it in range(a.iters + 3):
        held = P.allocator.alloc((a.tokens + 63) // 64)
        P.held_kv["bench"] = (held, a.tokens)
        torch.cuda.synchronize(d0)
        torch.cuda.synchronize(d1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream(d0))
        kv = P.export_kv("bench")
        req = D.add_prefilled(ids, 5, -1.0, kv, {"temperature": 0.0, "max_new_tokens": 2})
        torch.cuda.synchronize(d1)
        e1.record(torch.cuda.current_stream(d0))
        torch.cuda.synchronize(d0)
        if it >= 3:
            times.append(e0.elapsed_time(e1))
        P.release_kv("bench")
        D.abort_request(req.rid)
    nbytes = kv.numel() * kv.element_size()
    ms = sorted(times)[len(times) // 2]
    print(json.dumps({"tokens": a.tokens, "layers": a.layers, "kv_bytes": nbytes, "ms": ms, "gbs": nbytes / ms / 1e6,
                      "devices": [str(d0), str(d1)]}))


if __name__ == "__main__":
    _bench_handover()
