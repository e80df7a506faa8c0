"""Tinker-style multi-tenant LoRA training service.

Clients create *models* (a LoRA adapter slot on the shared base model), stream `forward_backward` batches with a named
loss (`cross_entropy, importance_sampling, ppo, cispo, dro`), call `optim_step` with their own Adam hyper-parameters,
sample from their current adapter and save / load / export it.  Reference: miles/tinker/runtime.py:46-206
(`MilesBackend`: slots, `forward_backward`, `optim_step`, `save_slot`, `export_slot`, `sample`), miles/tinker/core/*
(futures, per-model queues, scheduler) and miles/tinker/server/app.py (HTTP surface).

One base model with S adapter slots serves all tenants (`miles_b200.train.lora`): a batch carries a slot id per token,
so datums of different tenants can share a forward/backward; every slot has its own optimizer state
(`SlotOptimizer`).  Sampling runs on the engine that aliases the same model object, with the tenant's slot selected
per request.
"""
from __future__ import annotations

import asyncio
import itertools
import os
import time
from dataclasses import dataclass, field
from typing import Any

import torch

from ..models.qwen3 import ForwardMeta
from ..train import lora
from ..train.losses import TINKER_LOSSES, LossBatch


@dataclass
class TinkerModel:
    model_id: str
    slot: int
    rank: int
    created: float = field(default_factory=time.time)
    steps: int = 0
    pending_batches: int = 0


def _tokens_of(model_input: dict) -> list[int]:
    if "tokens" in model_input:
        return [int(t) for t in model_input["tokens"]]
    out: list[int] = []
    for ch in model_input.get("chunks", []):
        out.extend(int(t) for t in ch.get("tokens", []))
    return out


class TinkerService:
    def __init__(self, model, args, engine=None, pad_multiple: int = 1):
        assert getattr(model, "lora_adapters", None), "the base model needs LoRA slots (apply_lora with --lora-num-slots)"
        self.model, self.args, self.engine = model, args, engine
        self.num_slots = model.lora_adapters[0].slots
        self.free_slots = list(range(self.num_slots))
        self.models: dict[str, TinkerModel] = {}
        self.opt = lora.SlotOptimizer(model)
        self.futures: dict[str, Any] = {}
        self._fid = itertools.count()
        self.lock = asyncio.Lock()
        self.pad_multiple = pad_multiple
        self.device = next(model.parameters()).device

    # ---- model lifecycle -----------------------------------------------------------------------------
    def capabilities(self) -> dict:
        return {"supported_models": [{"model_name": getattr(self.args, "model_name", "base")}], "max_lora_rank": self.model.lora_adapters[0].rank,
                "free_slots": len(self.free_slots), "loss_fns": sorted(TINKER_LOSSES)}

    def create_model(self, model_id: str | None = None, lora_rank: int | None = None, seed: int = 0) -> TinkerModel:
        if not self.free_slots:
            raise RuntimeError("no free adapter slot")
        rank = self.model.lora_adapters[0].rank
        if lora_rank is not None and lora_rank > rank:
            raise ValueError(f"requested LoRA rank {lora_rank} exceeds the server's {rank}")
        slot = self.free_slots.pop(0)
        lora.zero_slot(self.model, slot, seed)
        self.opt.reset_slot(slot)
        mid = model_id or f"model-{slot}-{int(time.time() * 1000) % 10 ** 9}"
        self.models[mid] = TinkerModel(mid, slot, rank)
        return self.models[mid]

    def unload_model(self, model_id: str):
        m = self.models.pop(model_id)
        self.opt.reset_slot(m.slot)
        self.free_slots.append(m.slot)

    # ---- training ------------------------------------------------------------------------------------
    def _pack(self, datums: list[dict], slot: int):
        toks, pos, cu, slots = [], [], [0], []
        for d in datums:
            ids = _tokens_of(d["model_input"])
            toks += ids
            pos += list(range(len(ids)))
            cu.append(cu[-1] + len(ids))
            slots += [slot] * len(ids)
        real = len(toks)
        pad = (-real) % self.pad_multiple
        if pad:
            toks += [0] * pad
            pos += list(range(pad))
            cu.append(cu[-1] + pad)
            slots += [-1] * pad
        dev = self.device
        meta = ForwardMeta(positions=torch.tensor(pos, dtype=torch.int32, device=dev),
                           cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev),
                           max_seqlen=max(b - a for a, b in zip(cu[:-1], cu[1:])),
                           lora_slots=torch.tensor(slots, dtype=torch.long, device=dev))
        return torch.tensor(toks, dtype=torch.int32, device=dev), meta, real

    def _run(self, model_id: str, datums: list[dict], loss_fn: str, loss_fn_config: dict | None, backward: bool) -> dict:
        m = self.models[model_id]
        assert loss_fn in TINKER_LOSSES, f"unknown loss_fn {loss_fn}"
        tokens, meta, real = self._pack(datums, m.slot)
        dev = self.device
        lens = [len(_tokens_of(d["model_input"])) for d in datums]

        def cat(key, dtype=torch.float32, default=None):
            vals = []
            for d, n in zip(datums, lens):
                v = d.get("loss_fn_inputs", {}).get(key, default)
                if v is None:
                    return None
                v = v.get("data", v) if isinstance(v, dict) else v
                assert len(v) == n, f"{key} has {len(v)} entries for {n} tokens"
                vals += list(v)
            return torch.tensor(vals, dtype=dtype, device=dev)

        targets = cat("target_tokens", torch.int64)
        assert targets is not None, "loss_fn_inputs.target_tokens is required"
        weights = cat("weights")
        if weights is None:
            weights = torch.ones(real, device=dev)
        with torch.set_grad_enabled(backward):
            hidden = self.model(tokens, meta)[:real]
            lp, _ = self.model.log_probs(hidden, targets)
            seq_ids = torch.repeat_interleave(torch.arange(len(lens), device=dev), torch.tensor(lens, device=dev))
            batch = LossBatch(response_lengths=lens, loss_mask=(weights != 0).float(), seq_ids=seq_ids, advantages=cat("advantages"),
                              rollout_log_probs=cat("logprobs"), extra={"weights": weights, "loss_fn_config": loss_fn_config})
            loss, metrics = TINKER_LOSSES[loss_fn](self.args, batch, lp, None)
            if backward:
                loss.backward()
                m.pending_batches += 1
        outs = [{"logprobs": piece.tolist()} for piece in lp.detach().float().split(lens)]
        return {"loss_fn_output_type": loss_fn, "loss_fn_outputs": outs,
                "metrics": {"loss:sum": float(metrics["loss"]), "num_tokens": float(real)}}

    def forward_backward(self, model_id: str, datums: list[dict], loss_fn: str = "cross_entropy", loss_fn_config: dict | None = None):
        return self._run(model_id, datums, loss_fn, loss_fn_config, True)

    def forward(self, model_id: str, datums: list[dict], loss_fn: str = "cross_entropy", loss_fn_config: dict | None = None):
        return self._run(model_id, datums, loss_fn, loss_fn_config, False)

    def optim_step(self, model_id: str, adam_params: dict | None = None) -> dict:
        m = self.models[model_id]
        p = adam_params or {}
        self.opt.betas = (p.get("beta1", 0.9), p.get("beta2", 0.95))
        self.opt.eps, self.opt.wd = p.get("eps", 1e-8), p.get("weight_decay", 0.0)
        norm = self.opt.step(m.slot, lr=p.get("learning_rate", 1e-4), clip_grad=p.get("grad_clip_norm", 0.0))
        # gradients of other tenants' slots stay untouched: only this slot's slice is cleared
        for _, prm in self.opt.params:
            if prm.grad is not None:
                prm.grad[m.slot].zero_()
        m.steps += 1
        m.pending_batches = 0
        return {"metrics": {"grad_norm": norm, "step": m.steps}}

    # ---- weights -------------------------------------------------------------------------------------
    def save_weights(self, model_id: str, path: str, export_peft: bool = False) -> dict:
        m = self.models[model_id]
        os.makedirs(path, exist_ok=True)
        lora.save_adapter(self.model, path, slot=m.slot)
        torch.save({"optimizer": self.opt.state.get(m.slot), "steps": m.steps}, os.path.join(path, "optim.pt"))
        if export_peft:
            lora.export_peft(self.model, os.path.join(path, "peft"), slot=m.slot)
        return {"path": path}

    def load_weights(self, model_id: str, path: str, with_optimizer: bool = True) -> dict:
        m = self.models[model_id]
        lora.load_adapter(self.model, path, slot=m.slot)
        f = os.path.join(path, "optim.pt")
        if with_optimizer and os.path.exists(f):
            blob = torch.load(f, map_location="cpu", weights_only=False)
            if blob.get("optimizer") is not None:
                self.opt.state[m.slot] = blob["optimizer"]
            m.steps = blob.get("steps", 0)
        return {"path": path}

    # ---- sampling --------------------------------------------------------------------------------------
    def sample(self, model_id: str | None, prompt_tokens: list[int], sampling_params: dict | None = None, num_samples: int = 1) -> dict:
        assert self.engine is not None, "sampling needs an engine bound to the base model"
        slot = self.models[model_id].slot if model_id else -1
        sp = dict(sampling_params or {})
        if "max_tokens" in sp:
            sp["max_new_tokens"] = sp.pop("max_tokens")
        self.engine.lora_slot = slot                   # the engine tags its forward passes with this adapter slot
        seqs = []
        for i in range(num_samples):
            spi = dict(sp)
            if "seed" in spi:
                spi["seed"] = int(spi["seed"]) + i
            out = self.engine.generate(list(prompt_tokens), spi)
            seqs.append({"tokens": out["output_ids"], "logprobs": [p[0] for p in out["meta_info"]["output_token_logprobs"]],
                         "stop_reason": out["meta_info"]["finish_reason"]["type"]})
        self.engine.lora_slot = None
        return {"sequences": seqs}

    # ---- futures (the HTTP API is asynchronous: calls return a future id, results are retrieved later) --------
    def submit(self, fn, *a, **kw) -> str:
        fid = f"fut-{next(self._fid)}"
        try:
            self.futures[fid] = {"status": "done", "result": fn(*a, **kw)}
        except Exception as e:
            self.futures[fid] = {"status": "error", "error": f"{type(e).__name__}: {e}"}
        return fid

    def retrieve(self, fid: str) -> dict:
        return self.futures.pop(fid, {"status": "unknown"})
