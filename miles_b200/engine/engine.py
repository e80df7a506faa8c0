"""Rollout engine: continuous batching over a paged KV cache, token-in-token-out.

This is the in-repo equivalent of the external inference server the reference launches
(`python -m sglang.launch_server`, miles/backends/sglang_utils/sglang_engine.py:37-211) and talks to
over HTTP (miles/backends/sglang_utils/sglang_api_client.py:58-460).  The method names follow that
HTTP surface (`generate`, `pause_generation`, `continue_generation`, `flush_cache`,
`update_weights_from_tensor`, `release_memory_occupation`, `resume_memory_occupation`,
`update_weight_version` …); `miles_b200.engine.server` serves them over HTTP.

Scheduling: a step is either a prefill batch (new requests, up to `max_prefill_tokens`) or one decode
step for all running requests.  When blocks run out the youngest running request is retracted
(its blocks freed, it re-enters the waiting queue with prompt+output as the new prompt).
The engine can run on its own weights or *borrow the trainer's model object* (colocated mode): the
weight hand-over is then a pointer swap and `update_weights` is a version bump.
"""
from __future__ import annotations

import itertools
import threading
import time
import zlib
from collections import deque
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.qwen3 import ForwardMeta, Qwen3Model, build_model
from ..parallel.state import ParallelState
from ..types import encode_routed_experts
from .kv_cache import KVCache, make_allocator
from .sampler import SamplingParams, sample


@dataclass
class Request:
    rid: str
    input_ids: list[int]
    sampling: SamplingParams
    return_logprob: bool = True
    return_routed_experts: bool = False
    output_ids: list[int] = field(default_factory=list)
    output_logprobs: list[float] = field(default_factory=list)
    routed: list[np.ndarray] = field(default_factory=list)   # per forward pass: [tokens, L_moe, k]
    blocks: list[int] = field(default_factory=list)
    num_cached: int = 0            # tokens whose KV is in the cache
    finish_reason: dict | None = None
    weight_versions: list[list[int]] = field(default_factory=list)  # [version, num_tokens]
    arrival: float = field(default_factory=time.time)
    done: threading.Event = field(default_factory=threading.Event)
    retractions: int = 0
    seed: int = 0
    on_done: Any = None            # callable(Request), invoked from the engine thread
    stop_set: frozenset = frozenset()
    row: Any = None                # row in the decode runner's static buffers
    bt_len: int = 0
    logprob_start_len: int = -1    # ≥ 0: also return log-probs of the input tokens from this position on (scoring)
    input_logprobs: list[float] | None = None
    top_logprobs_num: int = 0      # > 0 with scoring: also the k most likely tokens (and their log-probs) at every scored position
    input_top_logprobs: list | None = None
    output_top_logprobs: list = field(default_factory=list)     # per generated token: the k most likely (log-prob, id, None)
    keep_kv: bool = False          # prefill / decode disaggregation: the cache blocks outlive the request until `release_kv`
    leader: Any = None             # request of the same prefill batch with identical tokens whose prompt KV this one shares
    cache_nodes: list = field(default_factory=list)   # prefix-cache nodes this request pins (their blocks head its block table)
    prefill_pos: int = 0           # tokens whose KV is in place (cached prefix + chunks already run); < len(all_ids) while prefilling
    chunk: tuple = (0, 0)          # token range [start, end) the next prefill step computes
    cached_tokens: int = 0         # prompt tokens whose KV was shared instead of recomputed

    @property
    def all_ids(self) -> list[int]:
        return self.input_ids + self.output_ids

    @property
    def num_tokens(self) -> int:
        return len(self.input_ids) + len(self.output_ids)

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def to_response(self, engine: "Engine", raw_routed: bool = False) -> dict:
        """The reply of `/generate`.  `raw_routed`: a caller in this process takes the routed experts as the int32 array
        itself instead of its base64 text (1.5 KB per token for 48 layers × top-8: the text form costs about a second per
        hundred thousand tokens to make and to parse)."""
        meta: dict[str, Any] = {
            "id": self.rid,
            "finish_reason": self.finish_reason,
            "prompt_tokens": len(self.input_ids),
            "completion_tokens": len(self.output_ids),
            "cached_tokens": self.cached_tokens,
            "weight_version": str(self.weight_versions[-1][0]) if self.weight_versions else str(engine.weight_version),
            "weight_version_spans": self.weight_versions,
        }
        if self.return_logprob:
            meta["output_token_logprobs"] = [(lp, t, None) for lp, t in zip(self.output_logprobs, self.output_ids)]
        if self.input_logprobs is not None:
            start = max(self.logprob_start_len, 0)
            # entry i scores input token start+i given everything before it; token 0 has no context (None)
            toks = self.input_ids[start:]
            lps = ([None] if start == 0 else []) + list(self.input_logprobs)
            meta["input_token_logprobs"] = [(lp, t, None) for lp, t in zip(lps, toks)]
            if self.input_top_logprobs is not None:
                meta["input_top_logprobs"] = ([None] if start == 0 else []) + self.input_top_logprobs
        if self.return_logprob and self.top_logprobs_num > 0:
            meta["output_top_logprobs"] = self.output_top_logprobs[:len(self.output_ids)]
        if self.return_routed_experts and self.routed:
            arr = np.concatenate(self.routed, axis=0)
            n = len(self.input_ids) + len(self.output_ids) - 1
            meta["routed_experts"] = arr[:n] if raw_routed else encode_routed_experts(arr[:n])
        text = engine.tokenizer.decode(self.output_ids) if engine.tokenizer is not None else ""
        return {"text": text, "output_ids": list(self.output_ids), "meta_info": meta}


class Engine:
    def __init__(self, cfg: ModelConfig, *, model: Qwen3Model | None = None, ps: ParallelState | None = None,
                 device="cpu", dtype=torch.bfloat16, num_blocks: int | None = None, block_size: int | None = None,
                 mem_fraction_static: float = 0.7, max_running_requests: int = 512, max_prefill_tokens: int = 16384,
                 max_context_len: int | None = None, eos_token_ids: list[int] | None = None, tokenizer=None,
                 seed: int = 0, use_cuda_graph: bool = True, record_routing: bool | None = None,
                 share_prompt_kv: bool = True, decode_steps_per_sync: int = 8, decode_steps_idle: int = 32,
                 prefix_cache: bool = True,
                 chunked_prefill_size: int | None = None):
        self.cfg = cfg
        self.ps = ps or ParallelState.single()
        self.device = torch.device(device)
        self.dtype = dtype
        self.model = model if model is not None else build_model(cfg, self.ps, dtype=dtype, device=device, seed=seed)
        self.owns_model = model is None
        self.block_size = block_size or (64 if self.device.type == "cuda" else 16)
        self.max_running = max_running_requests
        self.max_prefill_tokens = max_prefill_tokens
        self.max_context_len = max_context_len or cfg.max_position
        self.eos_token_ids = set(eos_token_ids or [])
        self.tokenizer = tokenizer
        self.mem_fraction_static = mem_fraction_static
        # requests of one prefill batch with identical tokens (the n samples of a prompt) run the prompt once: the full KV
        # blocks are shared by reference count, the partial last block is copied, the first token is sampled per request
        self.share_prompt_kv = share_prompt_kv
        # decode steps per host round trip on the CUDA runner (see `decode_runner`): a finished request may run up to
        # steps − 1 extra positions whose tokens are dropped; nothing waits on the host in between
        self.decode_steps_per_sync = max(1, int(decode_steps_per_sync))
        # with no request waiting for admission nothing gains from an early return to the scheduler: the round trip then
        # covers this many steps, and the host reads them back chunk by chunk while the GPU runs the rest
        self.decode_steps_idle = max(self.decode_steps_per_sync, int(decode_steps_idle))
        self._agreed_steps = 1
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        hkv = cfg.num_kv_heads // self.ps.tp_size
        if num_blocks is None:
            if self.device.type == "cuda":
                # blocks the caching allocator holds but no tensor uses (temporaries of the trainer's set-up) count as
                # used in mem_get_info: hand them back first, or the cache is sized from a fraction of what is really free
                torch.cuda.empty_cache()
                free, total = torch.cuda.mem_get_info(self.device)
                budget = int(free - (1.0 - mem_fraction_static) * total)
                budget = max(budget, 1 << 30)
                num_blocks = KVCache.blocks_for_budget(budget, len(self.model.layers), self.block_size, hkv, cfg.head_dim, dtype)
            else:
                num_blocks = 512
        lo, hi = self.model.layer_range
        self.kv = KVCache(hi - lo, num_blocks, self.block_size, hkv, cfg.head_dim, dtype, self.device,
                          layer_ids=list(range(lo, hi)))
        self.allocator = make_allocator(num_blocks)
        self.stateless = not getattr(self.model, "supports_kv_cache", True)
        # full KV blocks of finished prefills and finished requests stay in a block-granular radix tree: a later prompt that
        # starts with the same tokens (the next turn of a conversation, another sample of a prompt) computes only the rest
        from .prefix_cache import PrefixCache

        self.prefix_cache = PrefixCache(self.allocator, self.block_size) if (prefix_cache and not self.stateless) else None
        # prompts longer than this many new tokens are prefilled in pieces, one per step, each attending to the KV of the
        # pieces before it through the paged cache (None: a prompt is always one piece)
        self.chunked_prefill_size = int(chunked_prefill_size) if chunked_prefill_size else None
        self.prefilling: list[Request] = []          # requests between their first and last prefill piece (they hold blocks)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.weight_version = 0
        self.paused = False
        self.lock = threading.RLock()
        self._rid = itertools.count()
        self.seed = seed
        self._step_count = 0
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "steps": 0, "retractions": 0}
        self._loop_thread: threading.Thread | None = None
        self._stop_loop = False
        self._graphs: dict[int, Any] = {}
        # expert-parallel engines step in lockstep over the EP group (see `_step_lockstep`)
        self.lockstep_group = self.ps.ep_group if (self.ps.ep_size > 1 and cfg.is_moe) else None
        if self.lockstep_group is not None:
            from ..parallel.reloadable import REGISTRY

            REGISTRY.bind(self, "lockstep_group")
        self.local_done = True
        self.global_done = True
        self.held_kv: dict[str, tuple[list[int], int]] = {}     # finished `keep_kv` requests: (blocks, tokens with KV)
        self.runner = None
        self._agreed_bucket = 0
        # models whose mixers keep no paged KV (latent / linear attention of the other families) are served by scoring the
        # whole sequence again every step: correct for any block, quadratic in length — the functional path for those families
        if self.device.type == "cuda" and dtype == torch.bfloat16 and not self.stateless:
            from .decode_runner import DecodeRunner

            # expert-parallel dispatch over NCCL synchronises with the host, so it cannot be captured
            graphable = self.use_cuda_graph and (self.ps.ep_size == 1 or (self.ps.fabric is not None and self.ps.fused))
            self.runner = DecodeRunner(self, max_running_requests, graphable)

    # ---------------------------------------------------------------------------------------
    # request API
    # ---------------------------------------------------------------------------------------
    def add_request(self, input_ids: list[int], sampling_params: dict | SamplingParams | None = None,
                    return_logprob: bool = True, return_routed_experts: bool = False, rid: str | None = None,
                    on_done=None, logprob_start_len: int = -1, top_logprobs_num: int = 0, keep_kv: bool = False) -> Request:
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        with self.lock:
            rid = rid or f"req-{next(self._rid)}"
            req = Request(rid=rid, input_ids=list(input_ids), sampling=sp, return_logprob=return_logprob,
                          return_routed_experts=return_routed_experts and self.cfg.is_moe,
                          seed=(sp.seed if sp.seed is not None else (self.seed * 1000003 + zlib.crc32(rid.encode())) % (2 ** 31)),
                          on_done=on_done, logprob_start_len=int(logprob_start_len), top_logprobs_num=int(top_logprobs_num or 0),
                          keep_kv=bool(keep_kv))
            budget = self.max_context_len - len(input_ids)
            if budget <= 0 or sp.max_new_tokens <= 0:
                req.finish_reason = {"type": "length", "length": 0}
                req.done.set()
                if on_done is not None:
                    on_done(req)
                return req
            sp.max_new_tokens = min(sp.max_new_tokens, budget)
            req.stop_set = frozenset(sp.stop_token_ids) | (frozenset() if sp.ignore_eos else frozenset(self.eos_token_ids))
            self.requests[rid] = req
            self.waiting.append(req)
        return req

    # ---- prefill / decode disaggregation: a request's KV leaves this engine or arrives from another -------------------------
    def export_kv(self, rid: str) -> torch.Tensor:
        """KV of a finished `keep_kv` request as one tensor [layers, 2, tokens, kv heads, head dim] (a gather over its slots)."""
        with self.lock:
            blocks, n = self.held_kv[rid]
            slots = self._slot_tensor(blocks, n)
            layers = sorted(self.kv.layers)
            out = [torch.stack([self.kv.layers[l][0].flatten(0, 1).index_select(0, slots),
                                self.kv.layers[l][1].flatten(0, 1).index_select(0, slots)]) for l in layers]
            return torch.stack(out)

    def _slot_tensor(self, blocks: list[int], n: int) -> torch.Tensor:
        """Flat cache slots of positions 0 … n − 1 of a request with these blocks (built with tensor ops, not a Python loop)."""
        bs = self.block_size
        pos = torch.arange(n, dtype=torch.int64)
        return (torch.tensor(blocks, dtype=torch.int64)[pos // bs] * bs + pos % bs).to(self.device)

    def release_kv(self, rid: str):
        with self.lock:
            blocks, _ = self.held_kv.pop(rid, ([], 0))
            if blocks:
                self.allocator.release(blocks)

    def add_prefilled(self, input_ids: list[int], first_token: int, first_logprob: float, kv: torch.Tensor,
                      sampling_params: dict | SamplingParams | None = None, return_logprob: bool = True,
                      return_routed_experts: bool = False, routed: "np.ndarray | None" = None, rid: str | None = None,
                      on_done=None, seed: int | None = None) -> Request:
        """Continue a request whose prompt ran elsewhere: `kv` [layers, 2, len(input_ids), kv heads, head dim] is stored into
        freshly allocated blocks, `first_token` (sampled by the prefill engine) is its first output, decoding goes on here.
        Raises when the cache cannot take the prompt now (the caller retries or routes elsewhere)."""
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        assert not self.stateless, "engines that re-score the whole sequence keep no KV to receive"
        with self.lock:
            n = len(input_ids)
            assert kv.shape[2] == n and kv.shape[0] == len(self.kv.layers), (tuple(kv.shape), n, len(self.kv.layers))
            rid = rid or f"req-{next(self._rid)}"
            req = Request(rid=rid, input_ids=list(input_ids), sampling=sp, return_logprob=return_logprob,
                          return_routed_experts=return_routed_experts and self.cfg.is_moe,
                          seed=(seed if seed is not None else (sp.seed if sp.seed is not None else
                                                               (self.seed * 1000003 + zlib.crc32(rid.encode())) % (2 ** 31))),
                          on_done=on_done)
            sp.max_new_tokens = min(sp.max_new_tokens, self.max_context_len - n)
            req.stop_set = frozenset(sp.stop_token_ids) | (frozenset() if sp.ignore_eos else frozenset(self.eos_token_ids))
            blocks = self._alloc_blocks(self._blocks_needed(n + 1))
            if blocks is None:
                raise RuntimeError(f"no room for {n} prefilled tokens ({self._free_blocks()} blocks free)")
            req.blocks = blocks
            slots = self._slot_tensor(blocks, n)
            kv = kv.to(self.device)
            for i, l in enumerate(sorted(self.kv.layers)):
                kc, vc = self.kv.layers[l]
                kc.flatten(0, 1).index_copy_(0, slots, kv[i, 0].to(kc.dtype))
                vc.flatten(0, 1).index_copy_(0, slots, kv[i, 1].to(vc.dtype))
            req.num_cached = req.prefill_pos = n
            req.cached_tokens = n
            if routed is not None and req.return_routed_experts:
                req.routed.append(np.ascontiguousarray(routed[:n], dtype=np.int32))
            self.requests[rid] = req
            self.stats["received_kv_tokens"] = self.stats.get("received_kv_tokens", 0) + n
            self._append_token(req, int(first_token), float(first_logprob))
            if not req.finished:
                self.running.append(req)
                if self.runner is not None:
                    self.runner.attach(req)
        return req

    def abort_request(self, rid: str | None = None):
        """Abort one request (or all when rid is None); partial output is kept in the reply."""
        with self.lock:
            targets = [self.requests[rid]] if rid is not None and rid in self.requests else \
                (list(self.requests.values()) if rid is None else [])
            for r in targets:
                if not r.finished:
                    self._finish(r, {"type": "abort"})
            self.running = [r for r in self.running if not r.finished]
            self.waiting = deque(r for r in self.waiting if not r.finished)

    def generate(self, input_ids: list[int] | list[list[int]], sampling_params: dict | list[dict] | None = None,
                 return_logprob: bool = True, return_routed_experts: bool = False) -> dict | list[dict]:
        """Blocking generate; drives the step loop itself unless a background loop is running."""
        single = bool(input_ids) and isinstance(input_ids[0], int)
        batch = [input_ids] if single else list(input_ids)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * len(batch)
        reqs = [self.add_request(ids, dict(sp) if isinstance(sp, dict) else sp, return_logprob, return_routed_experts)
                for ids, sp in zip(batch, sps)]
        if self.lockstep_group is not None:
            self.begin_rollout()
            while True:
                if all(r.done.is_set() for r in reqs):
                    self.finish_rollout()
                if not self.step() and self.global_done:
                    break
        elif self._loop_thread is None:
            while not all(r.done.is_set() for r in reqs):
                if not self.step():
                    if self.paused:
                        time.sleep(0.001)
                    elif not self.waiting and not self.running and not self.prefilling:
                        break
        else:
            for r in reqs:
                r.done.wait()
        out = [r.to_response(self) for r in reqs]
        return out[0] if single else out

    # ---------------------------------------------------------------------------------------
    # control surface (names follow the HTTP endpoints the reference calls)
    # ---------------------------------------------------------------------------------------
    def pause_generation(self, mode: str = "retract"):
        """abort: finish running requests with reason abort; retract: push them back to waiting and free
        their KV; in_place: keep KV, just stop stepping."""
        with self.lock:
            self.paused = True
            if mode == "abort":
                self.abort_request(None)
            elif mode == "retract":
                for r in list(self.running) + list(self.prefilling):
                    self._retract(r)

    def continue_generation(self):
        with self.lock:
            self.paused = False

    def flush_cache(self) -> bool:
        with self.lock:
            if self.running or self.prefilling:
                return False
            if self.prefix_cache is not None:
                self.prefix_cache.reset()
            self.held_kv.clear()
            self.allocator.reset()
            return True

    def _cacheable(self, r: "Request") -> bool:
        """Requests whose prefix KV may come from / go to the prefix cache: plain generation.  Scoring requests need the
        hidden states of every prompt position, recorded routing needs every position's expert choice — both are computed
        only by running the whole prompt."""
        return self.prefix_cache is not None and r.logprob_start_len < 0 and not r.return_routed_experts

    def _invalidate_prefix_cache(self):
        """Cached KV belongs to the weights that computed it."""
        if self.prefix_cache is not None:
            self.prefix_cache.reset()

    def _alloc_blocks(self, n: int):
        """Allocate, evicting unpinned cached prefixes (least recently used first) when the free list is short."""
        if n > self.allocator.num_free and self.prefix_cache is not None:
            self.prefix_cache.evict(n - self.allocator.num_free)
        return self.allocator.alloc(n) if n > 0 else []

    def _free_blocks(self) -> int:
        return self.allocator.num_free + (self.prefix_cache.evictable() if self.prefix_cache is not None else 0)

    def update_weight_version(self, version: int):
        if int(version) != self.weight_version:
            self._invalidate_prefix_cache()
        self.weight_version = int(version)

    def get_weight_version(self) -> int:
        return self.weight_version

    def update_weights_from_tensor(self, named_tensors, weight_version: int | None = None, load_format: str | None = None):
        """Copy (or alias) tensors into the engine's model. Names are this package's parameter names for
        this rank's shard; HF-named full tensors go through `miles_b200.models.convert.load_hf_into`."""
        from ..models.convert import load_named_into_model

        with self.lock:
            load_named_into_model(self.model, named_tensors, self.cfg, self.ps)
            self._invalidate_prefix_cache()
            if weight_version is not None:
                self.weight_version = int(weight_version)
        return {"success": True}

    def update_weights_from_disk(self, model_path: str, weight_version: int | None = None):
        """Load an HF safetensors directory (full tensors, HF names) into this rank's shard.  A version directory of the
        delta protocol (`v{N}/manifest.json` under a delta root) is followed with a `DeltaReader` instead."""
        import os

        from ..checkpoint import hf_io
        from ..models.convert import load_named_into_model

        with self.lock:
            if os.path.exists(os.path.join(model_path, "manifest.json")):
                from ..weight_update.delta import DeltaReader

                root, leaf = os.path.split(os.path.normpath(model_path))
                rd = getattr(self, "_delta_reader", None)
                if rd is None or rd.root != root:
                    rd = self._delta_reader = DeltaReader(root)
                named = rd.update_to(int(leaf.lstrip("v"))).items()
            else:
                named = hf_io.load_hf_dir(model_path).items()
            load_named_into_model(self.model, named, self.cfg, self.ps)
            self._invalidate_prefix_cache()
            if weight_version is not None:
                self.weight_version = int(weight_version)
        return {"success": True}

    def init_weights_update_group(self, master_address: str, master_port: int, rank_offset: int, world_size: int,
                                  group_name: str = "weight_sync", backend: str | None = None):
        """Join the trainer's weight-broadcast group (disaggregated sync); this engine rank becomes
        `rank_offset + tp/ep-local rank` of it."""
        from ..weight_update import broadcast as bc

        backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
        local = getattr(self.ps, "rank_in_engine", 0)
        bc.make_group(backend, master_address, int(master_port), int(rank_offset) + local, int(world_size), name=group_name)
        return {"success": True}

    def update_weights_from_distributed(self, names, dtypes, shapes, group_name: str = "weight_sync",
                                        load_format: str | None = None, weight_version: int | None = None):
        """Receive one bucket (HF names, full tensors) broadcast by the trainer and load this rank's shard of it."""
        from ..models.convert import load_named_into_model
        from ..weight_update import broadcast as bc

        pg = bc.get_group(group_name)
        assert pg is not None, f"weight update group {group_name!r} was never initialised"
        meta = {"names": list(names), "dtypes": list(dtypes), "shapes": [list(s) for s in shapes]}
        named = bc.recv_bucket(pg, meta, load_format == "flattened_bucket", self.device)
        with self.lock:
            load_named_into_model(self.model, named, self.cfg, self.ps)
            if weight_version is not None:
                self.weight_version = int(weight_version)
        return {"success": True}

    def release_memory_occupation(self, tags: list[str] | None = None):
        tags = tags or ["kv_cache", "weights", "cuda_graph"]
        with self.lock:
            assert not self.running and not self.prefilling, "release_memory_occupation with requests in flight; pause (retract) first"
            if "kv_cache" in tags:
                if self.prefix_cache is not None:
                    self.prefix_cache.reset()              # the cached KV goes with the cache's memory
                self.kv.free()
                self.held_kv.clear()
                self.allocator.reset()
            if "cuda_graph" in tags:
                self._graphs.clear()
                if self.runner is not None:
                    self.runner.reset_graphs()
            if "weights" in tags and self.owns_model:
                self._weights_host = {n: p.data.to("cpu") for n, p in self.model.named_parameters()}
                for p in self.model.parameters():
                    p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            if torch.cuda.is_available():
                torch.cuda.empty_cache()

    def resume_memory_occupation(self, tags: list[str] | None = None):
        tags = tags or ["kv_cache", "weights", "cuda_graph"]
        with self.lock:
            if "weights" in tags and getattr(self, "_weights_host", None):
                for n, p in self.model.named_parameters():
                    p.data = self._weights_host[n].to(self.device)
                self._weights_host = None
            if "kv_cache" in tags and not self.kv.allocated:
                self.kv.allocate()

    def health(self) -> dict:
        return {"status": "ok", "running": len(self.running), "waiting": len(self.waiting), "prefilling": len(self.prefilling),
                "free_blocks": self.allocator.num_free, "weight_version": self.weight_version, "paused": self.paused,
                "cached_blocks": self.prefix_cache.num_nodes if self.prefix_cache is not None else 0}

    # ---------------------------------------------------------------------------------------
    # background loop (server mode)
    # ---------------------------------------------------------------------------------------
    def start_loop(self):
        if self._loop_thread is not None:
            return
        self._stop_loop = False

        def run():
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            while not self._stop_loop:
                if not self.step():
                    time.sleep(0.0005)

        self._loop_thread = threading.Thread(target=run, daemon=True, name="engine-loop")
        self._loop_thread.start()

    def stop_loop(self):
        self._stop_loop = True
        if self._loop_thread is not None:
            self._loop_thread.join(timeout=10)
            self._loop_thread = None

    # ---------------------------------------------------------------------------------------
    # scheduler
    # ---------------------------------------------------------------------------------------
    def _blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def _finish(self, r: Request, reason: dict):
        r.finish_reason = reason
        if self.runner is not None:
            self.runner.detach(r)
        if r in self.prefilling:
            self.prefilling.remove(r)
        if r.blocks:
            if self.prefix_cache is not None and self._cacheable(r) and reason.get("type") != "abort":
                # every position but the last sampled token has its KV written: the next turn of this conversation starts here
                n_kv = r.num_tokens - 1 if r.num_cached else r.prefill_pos       # num_cached > 0: the prefill completed
                full = max(0, n_kv) // self.block_size
                if full:
                    self.prefix_cache.insert(r.all_ids[: full * self.block_size], r.blocks[:full])
            if self.prefix_cache is not None and r.cache_nodes:
                self.prefix_cache.unpin(r.cache_nodes)
                r.cache_nodes = []
            if r.keep_kv and reason.get("type") != "abort":
                self.held_kv[r.rid] = (r.blocks, len(r.all_ids) - 1)       # every position but the last sampled token has KV
                while len(self.held_kv) > 4 * self.max_running:           # a caller that never came back: the oldest loans end
                    old = next(iter(self.held_kv))
                    self.allocator.release(self.held_kv.pop(old)[0])
            else:
                self.allocator.release(r.blocks)
            r.blocks = []
        self.requests.pop(r.rid, None)
        r.done.set()
        if r.on_done is not None:
            r.on_done(r)

    def _retract(self, r: Request):
        """Give the blocks back; the request restarts from a prefill of prompt+output."""
        if self.prefix_cache is not None and r.cache_nodes:
            self.prefix_cache.unpin(r.cache_nodes)
            r.cache_nodes = []
        if r.blocks:
            self.allocator.release(r.blocks)
        r.blocks, r.num_cached, r.prefill_pos = [], 0, 0
        if r in self.prefilling:
            self.prefilling.remove(r)
        r.retractions += 1
        if self.runner is not None:
            self.runner.detach(r)
        self.stats["retractions"] += 1
        if r in self.running:
            self.running.remove(r)
        self.waiting.appendleft(r)

    @torch.no_grad()
    def step(self) -> bool:
        """One scheduling step. Returns False when there was nothing to do."""
        # the engine batches arbitrary token counts, so it runs tensor parallelism without sequence sharding
        with self.lock, self.ps.no_sequence_parallel():
            if self.lockstep_group is not None:
                return self._step_lockstep()
            if self.paused or not self.kv.allocated:
                return False
            t0 = time.perf_counter()
            batch = self._schedule_prefill()
            if batch:
                self._run_prefill(batch)
                self.stats["prefill_s"] = self.stats.get("prefill_s", 0.0) + time.perf_counter() - t0
            elif self.running:
                k = self._decode_lookahead()
                if not self._ensure_decode_blocks(k):
                    return True
                n = len(self.running)
                self._agreed_steps = k
                self._run_decode()
                # wall time of decode steps by batch-size class (host bookkeeping included): where a rollout's time goes
                key = "decode_s_le8" if n <= 8 else "decode_s_le32" if n <= 32 else "decode_s_gt32"
                self.stats[key] = self.stats.get(key, 0.0) + time.perf_counter() - t0
                self.stats[key.replace("_s_", "_n_")] = self.stats.get(key.replace("_s_", "_n_"), 0) + self._agreed_steps
            else:
                return False
            self.stats["steps"] += 1
            self._step_count += 1
            self._debug_check("prefill" if batch else "decode")
            return True

    def _step_lockstep(self) -> bool:
        """Expert-parallel engines run the same kind of step at the same time because every MoE layer is a
        collective: ranks agree (one 3-int all-reduce) on prefill vs decode; a rank without work of that kind
        runs an empty batch.  `global_done` turns true once every rank called `finish_rollout()` and is idle."""
        import torch.distributed as dist

        batch = [] if self.paused else self._schedule_prefill()
        want_decode = bool(self.running) and not self.paused and not batch
        k = self._decode_lookahead() if want_decode else self._steps_wanted()
        if want_decode and not self._ensure_decode_blocks(k):
            want_decode = False
        # the decode batch bucket is agreed too (the largest any rank needs): with the same row count on every rank the
        # expert-parallel layers can bound what each rank receives by ep · rows · k instead of the buffer capacity
        bucket = self.runner.bucket_needed() if (self.runner is not None and want_decode) else 0
        # the number of steps per round trip is agreed as well: the smallest any rank can take (−k under MAX)
        flags = torch.tensor([int(bool(batch)), int(want_decode), int(not self.local_done), bucket, -k], dtype=torch.int32,
                             device=self.device if self.device.type == "cuda" else "cpu")
        t_agree = time.perf_counter()
        dist.all_reduce(flags, op=dist.ReduceOp.MAX, group=self.lockstep_group)
        any_prefill, any_decode, any_active, self._agreed_bucket, neg_k = (int(v) for v in flags.tolist())
        # the agreement itself plus the wait for the slowest rank's host
        self.stats["lockstep_agree_s"] = self.stats.get("lockstep_agree_s", 0.0) + time.perf_counter() - t_agree
        self.stats["lockstep_rounds"] = self.stats.get("lockstep_rounds", 0) + 1
        self._agreed_steps = max(1, -neg_k)
        self.global_done = not any_active and not any_prefill and not any_decode
        t0 = time.perf_counter()
        if any_prefill:
            self._run_prefill(batch)
            self.stats["prefill_s"] = self.stats.get("prefill_s", 0.0) + time.perf_counter() - t0
        elif any_decode:
            n = len(self.running)
            self._run_decode()
            key = "decode_s_le8" if n <= 8 else "decode_s_le32" if n <= 32 else "decode_s_gt32"
            self.stats[key] = self.stats.get(key, 0.0) + time.perf_counter() - t0
            self.stats[key.replace("_s_", "_n_")] = self.stats.get(key.replace("_s_", "_n_"), 0) + self._agreed_steps
        else:
            return False
        self.stats["steps"] += 1
        self._step_count += 1
        self._debug_check("prefill" if any_prefill else "decode")
        return True

    def _debug_check(self, where: str):
        """Debug build of the kernels only: after each engine step read what the index checks recorded and the device error
        flag, and stop with the step's context instead of going on with skipped accesses."""
        if self.device.type != "cuda":
            return
        from ..ops import cuda as K

        if not K.DEBUG_KERNELS:
            return
        rep, flag = K.bounds_report(), K.check_error_flag()
        if rep or flag:
            rows = [(r.rid, r.num_tokens, len(r.blocks), getattr(r, "row", None)) for r in self.running[:8]]
            raise RuntimeError(f"engine {where} step {self._step_count}: index checks {rep}, error flag {flag}, "
                               f"agreed steps {self._agreed_steps}, running {len(self.running)} {rows}")

    def check_fabric(self):
        """Raise if a peer-memory kernel of this process gave up a bounded wait (the step that followed is garbage)."""
        fab = getattr(self.ps, "fabric", None)
        if fab is not None:
            fab.check()

    dumper = None               # utils.dumper.DumperSwitch with the "inference" phase on (`attach_dumper`)

    def attach_dumper(self, switch):
        """Dump this engine's forwards under the inference phase; graphs cannot run Python hooks, so decode goes eager."""
        if switch is None or not switch.enabled("inference"):
            return
        self.dumper = switch
        switch.register(self.model)
        self.runner = None
        self.use_cuda_graph = False

    def _dumped_forward(self, toks, meta):
        if self.dumper is None:
            return self.model(toks, meta)
        with self.dumper.phase("inference"):
            hidden = self.model(toks, meta)
            self.dumper.step()
        return hidden

    def begin_rollout(self):
        import gc

        # lockstep ranks wait for the slowest host at every agreement: a cyclic-GC pause on one rank stalls all of them
        gc.collect()
        gc.disable()
        self.local_done = False
        self.global_done = False
        fab = getattr(self.ps, "fabric", None)
        if fab is not None:
            fab.phase_barrier(self.lockstep_group)      # host skew is absorbed here, not in a kernel's bounded wait
        if self.runner is not None and self.lockstep_group is not None and self.kv.allocated:
            self.runner.warmup()

    def finish_rollout(self):
        if not self.local_done:
            import gc

            gc.enable()
            self.check_fabric()
        self.local_done = True

    def _schedule_prefill(self) -> list[Request]:
        """Requests (each with the token range `chunk` it computes this step) for one prefill batch of at most
        `max_prefill_tokens` new tokens: first the next pieces of prompts that are mid-prefill, then newly admitted ones.
        A new request takes its longest cached prefix from the prefix cache; identical prompts of one batch share the
        first one's KV; with chunked prefill a prompt that does not fit the rest of the budget takes what is left."""
        batch, tokens = [], 0
        bs = self.block_size
        budget = self.max_prefill_tokens
        piece = self.chunked_prefill_size
        for r in self.prefilling:
            n = r.num_tokens
            take = min(n - r.prefill_pos, piece or n, max(budget - tokens, 0) if batch else (piece or n))
            if take <= 0:
                break
            r.chunk = (r.prefill_pos, r.prefill_pos + take)
            tokens += take
            batch.append(r)
        if len(batch) < len(self.prefilling):
            return batch                               # no room for newcomers while earlier prompts still wait for their pieces
        leaders: dict[tuple, Request] = {}
        share = self.share_prompt_kv and not self.stateless
        while self.waiting and len(self.running) + len(batch) < self.max_running:
            r = self.waiting[0]
            n = r.num_tokens
            key = None
            lead = None
            if share and r.logprob_start_len < 0:
                key = (n, hash(tuple(r.all_ids)))
                lead = leaders.get(key)
                if lead is not None and lead.all_ids != r.all_ids:
                    lead = None
            need = self._blocks_needed(n + 1)
            shared = (n // bs) if lead is not None else 0                  # full blocks of the leader's prompt
            hit = self.prefix_cache.match(r.all_ids, (n - 1) // bs) if (lead is None and self._cacheable(r)) else []
            cached = len(hit) * bs
            new_tokens = n - cached
            room = budget - tokens
            chunkable = piece is not None and lead is None and r.logprob_start_len < 0 and not self.stateless
            if chunkable:
                take = min(new_tokens, piece, room) if batch else min(new_tokens, piece)
                if take < new_tokens and take < bs:
                    break                              # not worth a piece smaller than a block: next step
            else:
                take = new_tokens
                if lead is None and batch and tokens + new_tokens > budget:
                    break
            # keep headroom so running requests can still grow by one block each
            if (need - shared - len(hit)) + len(self.running) > self._free_blocks() and (self.running or batch):
                break
            blocks = self._alloc_blocks(need - shared - len(hit))
            if blocks is None:
                if not self.running and not batch and not self.prefilling:
                    self.waiting.popleft()
                    self._finish(r, {"type": "abort", "message": "prompt does not fit in the KV cache"})
                    continue
                break
            self.waiting.popleft()
            if lead is not None:
                self.allocator.share(lead.blocks[:shared])
                r.blocks = lead.blocks[:shared] + blocks
                r.leader = lead
                r.cached_tokens = n
                r.chunk = (n, n)
            else:
                if hit:
                    r.cache_nodes = self.prefix_cache.acquire(r.all_ids, len(hit))      # pins the nodes, takes this request's references
                    self.stats["prefix_cache_hit_tokens"] = self.stats.get("prefix_cache_hit_tokens", 0) + cached
                r.blocks = [nd.block for nd in r.cache_nodes] + blocks
                r.leader = None
                r.cached_tokens = cached
                r.prefill_pos = cached
                r.chunk = (cached, cached + take)
                tokens += take
                if key is not None and cached + take == n:
                    leaders[key] = r                   # only a prompt that completes in this batch can lend its KV
            batch.append(r)
        return batch

    def _decode_lookahead(self) -> int:
        """Decode steps the next round trip may take: the configured count, bounded by what every running request may still
        generate and by the context limit (positions beyond either are never written)."""
        if self.runner is None or self.stateless or self.decode_steps_per_sync <= 1 or not self.running:
            return 1
        k = self._steps_wanted()
        if any(r.top_logprobs_num > 0 for r in self.running):
            return 1                       # the k most likely tokens are read from the step's logits on the host side
        for r in self.running:
            k = min(k, r.sampling.max_new_tokens - len(r.output_ids), self.max_context_len - r.num_tokens)
        return max(1, k)

    def _steps_wanted(self) -> int:
        if self.decode_steps_per_sync <= 1:
            return 1
        if self.lockstep_group is not None:
            return self.decode_steps_per_sync          # expert-parallel ranks keep the short round trip (one chunk per agreement)
        return self.decode_steps_per_sync if (self.waiting or self.prefilling) else self.decode_steps_idle

    def _ensure_decode_blocks(self, lookahead: int = 1) -> bool:
        """Every running request needs slots for its next `lookahead` tokens; retract the youngest on shortage."""
        bs = self.block_size
        while True:
            need = {id(r): max(0, self._blocks_needed(r.num_tokens + lookahead) - len(r.blocks)) for r in self.running}
            if sum(need.values()) <= self._free_blocks():
                for r in self.running:
                    if need[id(r)]:
                        r.blocks += self._alloc_blocks(need[id(r)])
                return True
            victim = max(self.running, key=lambda r: r.arrival)
            self._retract(victim)
            if not self.running:
                return False

    # ---------------------------------------------------------------------------------------
    # model execution
    # ---------------------------------------------------------------------------------------
    def _slots(self, r: Request, start: int, end: int) -> list[int]:
        bs = self.block_size
        return [r.blocks[p // bs] * bs + p % bs for p in range(start, end)]

    def _block_table(self, reqs: list[Request]) -> torch.Tensor:
        mx = max((len(r.blocks) for r in reqs), default=1)
        bt = torch.zeros(len(reqs), mx, dtype=torch.int32)
        for i, r in enumerate(reqs):
            bt[i, :len(r.blocks)] = torch.tensor(r.blocks, dtype=torch.int32)
        return bt.to(self.device)

    lora_slot: int | None = None     # multi-adapter serving: adapter slot applied to the engine's forward passes (−1 = base)

    def _lora_slots(self, n_tokens: int):
        if self.lora_slot is None:
            return None
        return torch.full((n_tokens,), int(self.lora_slot), dtype=torch.long, device=self.device)

    def enable_mxfp8_serving(self) -> int:
        """Serve the dense projections from MXFP8 copies (e4m3 payload + e8m0 scales per 1×32 block): allocates the
        quantised buffers, fills them from the current weights and registers them with the linear op.  Weight updates
        refresh them in one fused quantisation launch per bucket (`weight_update` with the engine's `quant_buffers`).
        Returns the number of bytes of quantised weights."""
        from ..ops import cuda as K
        from ..parallel.weight_sync import _skip_quant, fused_weight_sync

        assert self.device.type == "cuda", "MXFP8 serving needs the CUDA block-scaled GEMM"
        self.quant_buffers = {}
        total = 0
        for n, p in self.model.named_parameters():
            if p.dim() != 2 or p.dtype != torch.bfloat16 or _skip_quant(n, p) or p.shape[1] % 128 or p.shape[0] < 128:
                continue
            payload = torch.empty(p.numel(), dtype=torch.uint8, device=p.device)
            scales = torch.empty(p.numel() // 32, dtype=torch.uint8, device=p.device)
            self.quant_buffers[n] = (payload, scales)
            K.register_mxfp8_weight(p.data, payload, scales)
            total += payload.numel() + scales.numel()
        fused_weight_sync(type("A", (), {"model": self.model, "args": type("Args", (), {"update_weight_buffer_size": 512 << 20})()})(),
                          self, quant="mxfp8")
        return total

    def _run_prefill(self, batch: list[Request]):
        """Run the pieces scheduled by `_schedule_prefill`.  When every piece is a whole prompt starting from an empty cache
        the batch attends within its own tokens (packed variable-length attention); otherwise (a cached prefix, a later
        piece of a chunked prompt) the new tokens attend to their request's paged KV, which holds the earlier positions.
        Followers (identical tokens) take their leader's prompt KV — shared full blocks, a copy of the partial last block —
        and its last-position logits.  Requests whose prompt is complete after this step sample their first token."""
        lead_reqs = [r for r in batch if r.leader is None]
        toks, pos, slots, cu = [], [], [], [0]
        for r in lead_reqs:
            a, b = r.chunk
            ids = r.all_ids
            toks += ids[a:b]
            pos += list(range(a, b))
            slots += self._slots(r, a, b)
            cu.append(cu[-1] + (b - a))
        dev = self.device
        record = [] if any(r.return_routed_experts for r in batch) else None
        whole = all(r.chunk[0] == 0 for r in lead_reqs)
        if whole or self.stateless:
            meta = ForwardMeta(
                positions=torch.tensor(pos, dtype=torch.int32, device=dev),
                cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev),
                max_seqlen=max((r.chunk[1] for r in lead_reqs), default=0),
                kv_cache=None if self.stateless else self.kv.layers,
                slot_mapping=None if self.stateless else torch.tensor(slots, dtype=torch.int64, device=dev),
                record_topk=record, lora_slots=self._lora_slots(len(toks)))
        else:
            # keys of request i: positions [0, end_i) read from its blocks; queries: its new tokens [start_i, end_i)
            gather = []
            cu_k = [0]
            for r in lead_reqs:
                gather += self._slots(r, 0, r.chunk[1])
                cu_k.append(cu_k[-1] + r.chunk[1])
            meta = ForwardMeta(
                positions=torch.tensor(pos, dtype=torch.int32, device=dev), cu_seqlens=None,
                max_seqlen=max((r.chunk[1] - r.chunk[0] for r in lead_reqs), default=0),
                kv_cache=self.kv.layers, block_table=self._block_table(lead_reqs),
                seq_lens=torch.tensor([r.chunk[1] for r in lead_reqs], dtype=torch.int32, device=dev),
                q_lens=torch.tensor([r.chunk[1] - r.chunk[0] for r in lead_reqs], dtype=torch.int32, device=dev),
                slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev),
                record_topk=record, lora_slots=self._lora_slots(len(toks)))
            meta.extend = {"cu_q": torch.tensor(cu, dtype=torch.int32, device=dev), "cu_k": torch.tensor(cu_k, dtype=torch.int32, device=dev),
                           "kv_slots": torch.tensor(gather, dtype=torch.int64, device=dev),
                           "max_k": max((r.chunk[1] for r in lead_reqs), default=0)}
            self.stats["extend_tokens"] = self.stats.get("extend_tokens", 0) + len(toks)
        self.stats["h2d_bytes"] = self.stats.get("h2d_bytes", 0) + 4 * len(toks) * 2 + 4 * len(cu) + 8 * len(slots)
        hidden = self._dumped_forward(torch.tensor(toks, dtype=torch.int32, device=dev), meta)
        if not batch:
            return
        hidden = self.ps.sp_gather(hidden)
        self.stats["prefill_tokens"] += len(toks)
        span = {id(r): (a, b) for r, a, b in zip(lead_reqs, cu[:-1], cu[1:])}
        for r, a, b in zip(lead_reqs, cu[:-1], cu[1:]):
            if r.logprob_start_len >= 0 and r.input_logprobs is None and r.retractions == 0:
                # score the prompt: row p predicts token p+1 (temperature 1, the teacher / reference distribution)
                n_in = len(r.input_ids)
                lo = max(r.logprob_start_len - 1, 0)
                rows = torch.arange(a + lo, a + n_in - 1, device=dev)
                tgt = torch.tensor(r.input_ids[lo + 1:n_in], dtype=torch.int64, device=dev)
                lp, _ = self.model.log_probs(hidden[rows], tgt) if len(tgt) else (torch.empty(0), None)
                r.input_logprobs = [float(x) for x in lp.float().tolist()]
                if r.top_logprobs_num > 0 and len(tgt):
                    tops = []
                    for c0 in range(0, rows.numel(), 512):          # full-vocabulary rows, 512 at a time
                        lg = torch.log_softmax(self.model.logits(hidden[rows[c0:c0 + 512]]).float(), dim=-1)
                        v, i = lg.topk(min(r.top_logprobs_num, lg.shape[-1]), dim=-1)
                        tops += [[(float(x), int(y), None) for x, y in zip(vr, ir)] for vr, ir in zip(v.tolist(), i.tolist())]
                    r.input_top_logprobs = tops
        followers = [r for r in batch if r.leader is not None]
        if followers:
            self._copy_tail_blocks(followers)
            self.stats["shared_prompt_tokens"] = self.stats.get("shared_prompt_tokens", 0) + sum(r.cached_tokens for r in followers)
        if record is not None:
            rec = torch.stack(record, dim=1).cpu().numpy().astype(np.int32)  # [T, L_moe, k]
            self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + rec.nbytes
            for r in batch:
                if r.return_routed_experts:
                    src = r.leader if r.leader is not None else r
                    a, b = span[id(src)]
                    start = src.chunk[0]
                    # rows [a, b) are tokens [start, end); after a retraction the request already holds its first `have` rows
                    have = sum(x.shape[0] for x in r.routed)
                    r.routed.append(rec[a + max(have - start, 0):b])
        done, lead_row = [], {}
        for i, r in enumerate(lead_reqs):
            r.prefill_pos = r.chunk[1]
            if r.prefill_pos >= r.num_tokens:
                lead_row[id(r)] = len(done)
                done.append(i)
                if r in self.prefilling:
                    self.prefilling.remove(r)
                if self._cacheable(r):
                    full = r.num_tokens // self.block_size
                    if full:
                        # the request goes on using these blocks: pin the nodes that own them until it finishes
                        held = set(map(id, r.cache_nodes))
                        fresh = [nd for nd in self.prefix_cache.insert(r.all_ids[: full * self.block_size], r.blocks[:full])
                                 if id(nd) not in held]
                        self.prefix_cache.pin(fresh)
                        r.cache_nodes = r.cache_nodes + fresh
            elif r not in self.prefilling:
                self.prefilling.append(r)
        finished_batch = [r for r in batch if (r.leader if r.leader is not None else r).prefill_pos >= r.num_tokens]
        if not finished_batch:
            return
        last = torch.tensor([cu[i + 1] - 1 for i in done], dtype=torch.int64, device=dev)
        logits = self.model.logits(hidden[last])
        for r in finished_batch:
            r.num_cached = r.num_tokens
            r.prefill_pos = r.num_tokens
        if followers or len(done) != len(finished_batch):
            rows = torch.tensor([lead_row[id(r.leader if r.leader is not None else r)] for r in finished_batch], dtype=torch.int64, device=dev)
            logits = logits[rows]
        for r in batch:
            r.leader = None
        self._sample_and_append(finished_batch, logits)
        for r in finished_batch:
            if not r.finished and r not in self.running:
                self.running.append(r)
                if self.runner is not None:
                    self.runner.attach(r)

    def _copy_tail_blocks(self, followers: list[Request]):
        """Followers own their last (partial) prompt block: copy the leader's partial block into it, all followers and
        all layers' K and V in one indexed copy per tensor."""
        bs = self.block_size
        src, dst = [], []
        for r in followers:
            n = r.num_tokens
            if n % bs:
                src.append(r.leader.blocks[n // bs])
                dst.append(r.blocks[n // bs])
        if not src:
            return
        s_idx = torch.tensor(src, dtype=torch.int64, device=self.device)
        d_idx = torch.tensor(dst, dtype=torch.int64, device=self.device)
        for kc, vc in self.kv.layers.values():
            kc[d_idx] = kc[s_idx]
            vc[d_idx] = vc[s_idx]

    def _run_decode(self):
        if self.stateless:
            reqs = list(self.running)
            self.stats["decode_tokens"] += len(reqs)
            for r in reqs:
                r.chunk = (0, r.num_tokens)             # the whole sequence, every step
            self._run_prefill(reqs)                       # scores every sequence from its first token; appends one token each
            self.stats["prefill_tokens"] -= sum(r.num_tokens - 1 for r in reqs)
            self.running = [r for r in self.running if not r.finished]
            return
        if self.runner is not None:
            return self._run_decode_static()
        reqs = self.running
        dev = self.device
        toks = [r.all_ids[-1] for r in reqs]
        pos = [r.num_tokens - 1 for r in reqs]
        slots = [self._slots(r, p, p + 1)[0] for r, p in zip(reqs, pos)]
        record = [] if any(r.return_routed_experts for r in reqs) else None
        meta = ForwardMeta(
            positions=torch.tensor(pos, dtype=torch.int32, device=dev), cu_seqlens=None, max_seqlen=1,
            kv_cache=self.kv.layers, block_table=self._block_table(reqs),
            seq_lens=torch.tensor([p + 1 for p in pos], dtype=torch.int32, device=dev),
            slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev), record_topk=record,
            lora_slots=self._lora_slots(len(toks)))
        hidden = self._dumped_forward(torch.tensor(toks, dtype=torch.int32, device=dev), meta)
        if not reqs:
            return
        hidden = self.ps.sp_gather(hidden)
        logits = self.model.logits(hidden)
        self.stats["decode_tokens"] += len(toks)
        if record is not None:
            rec = torch.stack(record, dim=1).cpu().numpy().astype(np.int32)
            for i, r in enumerate(reqs):
                if r.return_routed_experts:
                    r.routed.append(rec[i:i + 1])
        self._sample_and_append(reqs, logits)
        self.running = [r for r in reqs if not r.finished]

    def _run_decode_static(self):
        """CUDA path: static buffers + (optionally) a CUDA graph per batch bucket; see `decode_runner`."""
        reqs = self.running
        steps = self._agreed_steps
        tok, lp, routed = self.runner.step(reqs, self._step_count,
                                           min_bucket=self._agreed_bucket if self.lockstep_group is not None else 0, steps=steps)
        if steps == 1:
            self.stats["decode_tokens"] += len(reqs)
            if any(r.top_logprobs_num > 0 for r in reqs):
                self._collect_top_logprobs(reqs, self.runner.last_logits, [r.row for r in reqs])
            for r in reqs:
                row = r.row
                if routed is not None and r.return_routed_experts:
                    r.routed.append(routed[row:row + 1].copy())
                self._append_token(r, int(tok[row]), float(lp[row]))
        else:
            rows = [(r, r.row) for r in reqs]      # `_finish` detaches the row; keep it for the remaining sub-steps
            ch = self.runner.chunk_steps
            for k0 in range(0, steps, ch):
                k1 = min(steps, k0 + ch)
                self.runner.wait_step(k1 - 1)      # a chunk of steps at a time; the GPU is running the later chunks meanwhile
                for r, row in rows:
                    if r.finished:
                        continue                   # what a row produced after its stop token / limit is dropped
                    if routed is not None and r.return_routed_experts:
                        # [tokens, layers, top-k], one copy per chunk and row, in place before a token can finish the request
                        # (a waiter may read the result at once); rows past the last token are cut off with the output
                        r.routed.append(routed[k0:k1, row].copy())
                    k = k0
                    while k < k1 and not r.finished:
                        self._append_token(r, int(tok[k, row]), float(lp[k, row]))
                        k += 1
                    self.stats["decode_tokens"] += k - k0
            self.stats["decode_extra_steps"] = self.stats.get("decode_extra_steps", 0) + steps - 1
        self.running = [r for r in reqs if not r.finished]

    def _append_token(self, r: Request, t: int, l: float):
        if not (0 <= t < self.cfg.vocab_size) or l != l:
            # a non-finite hidden state; stop here rather than feed the id to the next step's embedding lookup
            raise RuntimeError(f"engine step {self._step_count}: request {r.rid} sampled id {t} with log-prob {l} "
                               f"(context {r.num_tokens} tokens, {len(self.running)} running)")
        r.output_ids.append(t)
        r.output_logprobs.append(l)
        if r.weight_versions and r.weight_versions[-1][0] == self.weight_version:
            r.weight_versions[-1][1] += 1
        else:
            r.weight_versions.append([self.weight_version, 1])
        if t in r.stop_set:
            self._finish(r, {"type": "stop", "matched": t})
        elif len(r.output_ids) >= r.sampling.max_new_tokens:
            self._finish(r, {"type": "length", "length": len(r.output_ids)})

    def _collect_top_logprobs(self, reqs: list[Request], logits: torch.Tensor, rows: list[int]):
        """`top_logprobs_num` of a request: the k most likely next tokens under its sampling temperature, appended before the
        sampled token is (the entry belongs to the token about to be appended)."""
        for r, row in zip(reqs, rows):
            if r.top_logprobs_num <= 0:
                continue
            t = r.sampling.temperature if r.sampling.temperature > 0 else 1.0
            lg = torch.log_softmax(logits[row].float() / t, dim=-1)
            v, i = lg.topk(min(r.top_logprobs_num, lg.shape[-1]))
            r.output_top_logprobs.append([(float(x), int(y), None) for x, y in zip(v.tolist(), i.tolist())])

    def _sample_and_append(self, reqs: list[Request], logits: torch.Tensor):
        dev = self.device
        temp = torch.tensor([r.sampling.temperature for r in reqs], dtype=torch.float32, device=dev)
        top_p = torch.tensor([r.sampling.top_p for r in reqs], dtype=torch.float32, device=dev)
        top_k = torch.tensor([r.sampling.top_k for r in reqs], dtype=torch.int64, device=dev)
        # the random stream of a request depends on its seed and its own token count only, never on what else is batched
        seeds = torch.tensor([(r.seed * 1000003 + len(r.output_ids)) & 0x7FFFFFFFFFFFFFFF for r in reqs], dtype=torch.int64,
                             device=dev)
        tok, lp = sample(logits.float(), temp, top_p, top_k, seeds=seeds, step=0)
        self._collect_top_logprobs(reqs, logits, list(range(len(reqs))))
        tok_l, lp_l = tok.tolist(), lp.tolist()
        self.stats["h2d_bytes"] = self.stats.get("h2d_bytes", 0) + 24 * len(reqs)
        self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + 12 * len(reqs)
        for r, t, l in zip(reqs, tok_l, lp_l):
            self._append_token(r, int(t), float(l))
