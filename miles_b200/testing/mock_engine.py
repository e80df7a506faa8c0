"""A scripted stand-in for the rollout engine, with the engine's Python API and (through `engine.server`) its HTTP
surface — the counterpart of the mock SGLang server/engine the reference ships for tests
(miles/utils/test_utils/mock_sglang_server.py and friends).

It needs no model: output tokens are a deterministic function of the prompt and the step, log-probs are fixed, finish
reasons follow `max_new_tokens` / stop tokens.  Latency, failures and aborts can be scripted, which is what rollout,
router, weight-update-session and fault-tolerance tests need.
"""
from __future__ import annotations

import base64
import itertools
import threading
import time
import zlib
from dataclasses import dataclass, field
from typing import Any

import numpy as np


@dataclass
class MockRequest:
    rid: str
    input_ids: list[int]
    max_new_tokens: int
    stop: frozenset
    output_ids: list[int] = field(default_factory=list)
    finish_reason: dict | None = None
    done: threading.Event = field(default_factory=threading.Event)
    on_done: Any = None
    return_routed_experts: bool = False
    weight_versions: list[list[int]] = field(default_factory=list)

    def to_response(self, engine, raw_routed: bool = False) -> dict:
        meta = {"id": self.rid, "finish_reason": self.finish_reason, "prompt_tokens": len(self.input_ids),
                "completion_tokens": len(self.output_ids), "cached_tokens": 0,
                "weight_version": str(engine.weight_version), "weight_version_spans": self.weight_versions,
                "output_token_logprobs": [(engine.logprob, t, None) for t in self.output_ids]}
        if self.return_routed_experts and engine.num_moe_layers:
            n = len(self.input_ids) + len(self.output_ids) - 1
            arr = (np.arange(n * engine.num_moe_layers * engine.moe_topk, dtype=np.int32) % engine.num_experts
                   ).reshape(n, engine.num_moe_layers, engine.moe_topk)
            meta["routed_experts"] = base64.b64encode(arr.tobytes()).decode()
        return {"text": " ".join(map(str, self.output_ids)), "output_ids": list(self.output_ids), "meta_info": meta}


class MockEngine:
    def __init__(self, vocab_size: int = 1000, tokens_per_step: int = 1, step_latency_s: float = 0.0, logprob: float = -1.0,
                 num_moe_layers: int = 0, moe_topk: int = 0, num_experts: int = 0, fail_after: int | None = None):
        self.vocab_size, self.tokens_per_step, self.step_latency_s, self.logprob = vocab_size, tokens_per_step, step_latency_s, logprob
        self.num_moe_layers, self.moe_topk, self.num_experts = num_moe_layers, moe_topk, num_experts
        self.fail_after = fail_after
        self.requests: dict[str, MockRequest] = {}
        self.running: list[MockRequest] = []
        self.weight_version = 0
        self.paused = False
        self.lock = threading.RLock()
        self._rid = itertools.count()
        self.calls: list[tuple] = []          # every control call, for assertions on session framing
        self.lockstep_group = None
        self.global_done = True
        self.cfg = type("Cfg", (), {"is_moe": num_moe_layers > 0, "moe_topk": moe_topk})()
        self.model = type("M", (), {"num_moe_layers": num_moe_layers})()
        self.tokenizer = None
        self.device = "cpu"
        self._loop: threading.Thread | None = None
        self._stop_loop = False
        self.steps = 0

    # ---- request API -------------------------------------------------------------------------------
    def next_token(self, req: MockRequest) -> int:
        seed = zlib.crc32(bytes(str((req.input_ids[-4:], len(req.output_ids))), "utf8"))
        return 3 + seed % (self.vocab_size - 3)

    def add_request(self, input_ids, sampling_params=None, return_logprob=True, return_routed_experts=False, rid=None,
                    on_done=None, logprob_start_len=-1):
        sp = dict(sampling_params or {})
        with self.lock:
            rid = rid or f"mock-{next(self._rid)}"
            r = MockRequest(rid, list(input_ids), int(sp.get("max_new_tokens", 16)), frozenset(sp.get("stop_token_ids") or []),
                            on_done=on_done, return_routed_experts=return_routed_experts)
            self.requests[rid] = r
            if r.max_new_tokens <= 0:
                self._finish(r, {"type": "length", "length": 0})
            else:
                self.running.append(r)
        return r

    def _finish(self, r: MockRequest, reason: dict):
        r.finish_reason = reason
        r.done.set()
        if r.on_done is not None:
            r.on_done(r)

    def step(self) -> bool:
        with self.lock:
            if self.paused or not self.running:
                return False
            if self.fail_after is not None and self.steps >= self.fail_after:
                raise RuntimeError("mock engine failure (scripted)")
            if self.step_latency_s:
                time.sleep(self.step_latency_s)
            self.steps += 1
            for r in list(self.running):
                for _ in range(self.tokens_per_step):
                    t = self.next_token(r)
                    r.output_ids.append(t)
                    if not r.weight_versions or r.weight_versions[-1][0] != self.weight_version:
                        r.weight_versions.append([self.weight_version, 0])
                    r.weight_versions[-1][1] += 1
                    if t in r.stop:
                        self._finish(r, {"type": "stop", "matched": t})
                        break
                    if len(r.output_ids) >= r.max_new_tokens:
                        self._finish(r, {"type": "length", "length": len(r.output_ids)})
                        break
            self.running = [r for r in self.running if r.finish_reason is None]
            return True

    def generate(self, input_ids, sampling_params=None, return_logprob=True, return_routed_experts=False):
        single = bool(input_ids) and isinstance(input_ids[0], int)
        reqs = [self.add_request(ids, sampling_params, return_logprob, return_routed_experts)
                for ids in ([input_ids] if single else input_ids)]
        while not all(r.done.is_set() for r in reqs):
            if not self.step() and self.paused:
                time.sleep(0.001)
        out = [r.to_response(self) for r in reqs]
        return out[0] if single else out

    def abort_request(self, rid=None):
        with self.lock:
            for r in list(self.running):
                if rid is None or r.rid == rid:
                    self._finish(r, {"type": "abort"})
            self.running = [r for r in self.running if r.finish_reason is None]
            self.calls.append(("abort_request", rid))

    # ---- control surface -----------------------------------------------------------------------------
    def _record(self, name, *a):
        self.calls.append((name, *a))
        return {"success": True}

    def begin_rollout(self):
        pass

    def finish_rollout(self):
        pass

    def start_loop(self):
        if self._loop is None:
            def run():
                while not self._stop_loop:
                    if not self.step():
                        time.sleep(0.001)
            self._loop = threading.Thread(target=run, daemon=True, name="mock-engine")
            self._loop.start()

    def pause_generation(self, mode="retract"):
        self.paused = True
        if mode == "abort":
            self.abort_request(None)
        return self._record("pause_generation", mode)

    def continue_generation(self):
        self.paused = False
        return self._record("continue_generation")

    def flush_cache(self):
        self._record("flush_cache")
        return True

    def update_weight_version(self, v):
        self.weight_version = int(v)
        return self._record("update_weight_version", int(v))

    def get_weight_version(self):
        return self.weight_version

    def update_weights_from_tensor(self, named, weight_version=None, load_format=None):
        if weight_version is not None:
            self.weight_version = int(weight_version)
        return self._record("update_weights_from_tensor", len(list(named)), load_format)

    def update_weights_from_disk(self, path, weight_version=None):
        return self._record("update_weights_from_disk", path)

    def release_memory_occupation(self, tags=None):
        return self._record("release_memory_occupation", tuple(tags or ()))

    def resume_memory_occupation(self, tags=None):
        return self._record("resume_memory_occupation", tuple(tags or ()))
