"""Inference controller: owns the rollout engines of every served model, their memory state and their health.

Reference: miles/ray/rollout/inference_controller.py:45-416 (+ rollout_server.py, server_cell.py): one `RolloutServer`
per model → one `ServerCell` per engine; lock-disciplined offload / onload (colocated memory hand-over), `start/end
_update_weights` framing, a reconcile tick that restarts or re-admits cells, a separate evaluation fleet;
miles/backends/sglang_utils/sglang_config.py:144-400 (multi-model `--sglang-config`: server groups of type
regular / prefill / decode / placeholder with per-group overrides) and sglang_engine.py:37-211 (launch command).

Engines are objects with the engine API (`miles_b200.engine.Engine`, `weight_update.broadcast.RemoteEngine`, or the
mock engine); the controller never assumes they live in this process.
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass, field
from typing import Any

import yaml

from ..ft.controller import EngineHealthChecker

GROUP_TYPES = ("regular", "prefill", "decode", "placeholder")


@dataclass
class ServerGroup:
    worker_type: str = "regular"
    num_gpus: int = 1
    num_gpus_per_engine: int = 1
    overrides: dict = field(default_factory=dict)       # engine kwargs of this group (mem fraction, parallel sizes, …)

    @property
    def num_engines(self) -> int:
        return 0 if self.worker_type == "placeholder" else self.num_gpus // self.num_gpus_per_engine


@dataclass
class ModelServingConfig:
    name: str
    model_path: str | None = None
    groups: list[ServerGroup] = field(default_factory=list)
    eval_only: bool = False
    update_weights: bool = True                          # frozen models (reward / teacher) skip weight sync


def load_serving_config(path_or_dict) -> list[ModelServingConfig]:
    """`--engine-config file.yaml`: {models: [{name, model_path, eval_only, update_weights, server_groups: [{worker_type,
    num_gpus, num_gpus_per_engine, overrides}]}]}"""
    spec = path_or_dict
    if isinstance(spec, str):
        with open(spec) as f:
            spec = yaml.safe_load(f)
    out = []
    for m in spec["models"]:
        groups = []
        for g in m.get("server_groups", [{"worker_type": "regular"}]):
            wt = g.get("worker_type", "regular")
            assert wt in GROUP_TYPES, f"unknown worker_type {wt}"
            per = g.get("num_gpus_per_engine", 1)
            n = g.get("num_gpus", per)
            assert n % per == 0, f"{m['name']}: num_gpus {n} is not a multiple of num_gpus_per_engine {per}"
            groups.append(ServerGroup(wt, n, per, dict(g.get("overrides") or {})))
        if any(g.worker_type == "prefill" for g in groups) != any(g.worker_type == "decode" for g in groups):
            raise ValueError(f"{m['name']}: prefill and decode groups come in pairs (PD disaggregation)")
        out.append(ModelServingConfig(m["name"], m.get("model_path"), groups, m.get("eval_only", False), m.get("update_weights", True)))
    return out


def engine_launch_cmd(model: ModelServingConfig, group: ServerGroup, port: int = 30000, extra: dict | None = None) -> list[str]:
    """Command line of one engine server of `group` (`python -m miles_b200.engine.server …`); `{port}` style placeholders
    are filled by the worker planner."""
    kw = {"tp": group.num_gpus_per_engine, **group.overrides, **(extra or {})}
    cmd = ["python", "-m", "miles_b200.engine.server", "--port", str(port)]
    if model.model_path:
        cmd += ["--hf-checkpoint", model.model_path]
    if group.worker_type in ("prefill", "decode"):
        cmd += ["--disaggregation-mode", group.worker_type]
    for k, v in kw.items():
        flag = "--" + k.replace("_", "-")
        if isinstance(v, bool):
            if v:
                cmd.append(flag)
        else:
            cmd += [flag, str(v)]
    return cmd


class ContextLock:
    """A lock that records which operation holds it: offload/onload/update are mutually exclusive, and a second request
    for the state the engines are already in is a no-op instead of a deadlock."""

    def __init__(self):
        self._lock = threading.Lock()
        self.holder: str | None = None

    @contextlib.contextmanager
    def hold(self, what: str):
        with self._lock:
            self.holder = what
            try:
                yield
            finally:
                self.holder = None


@dataclass
class ServerCell:
    engine: Any
    model: str
    group: ServerGroup
    state: str = "alive"             # alive | offloaded | unhealthy


class InferenceController:
    def __init__(self, cells: list[ServerCell], probe=None, health_threshold: int = 3):
        self.cells = cells
        self.lock = ContextLock()
        self.weight_version = 0
        self.updating = False
        self.health = EngineHealthChecker([c.engine for c in cells], probe or (lambda e: True), health_threshold,
                                          on_unhealthy=self._on_unhealthy, on_recovered=self._on_recovered)

    # ---- selection ---------------------------------------------------------------------------------
    def engines(self, model: str | None = None, include_eval: bool = False, only_trainable: bool = False) -> list:
        out = []
        for c in self.cells:
            if c.state == "unhealthy" or (model is not None and c.model != model):
                continue
            out.append(c.engine)
        return out

    def _cell_of(self, engine):
        return next(c for c in self.cells if c.engine is engine)

    def _on_unhealthy(self, engine):
        self._cell_of(engine).state = "unhealthy"

    def _on_recovered(self, engine):
        c = self._cell_of(engine)
        c.state = "alive"
        # a re-admitted engine missed weight updates: bring its version label in line; the updater re-syncs it
        if hasattr(engine, "get_weight_version") and engine.get_weight_version() != self.weight_version:
            c.state = "stale"

    def tick(self):
        """One reconcile pass: probe engines, quarantine / re-admit."""
        self.health.check_once()
        return {c.model + f"#{i}": c.state for i, c in enumerate(self.cells)}

    def stale_engines(self) -> list:
        return [c.engine for c in self.cells if c.state == "stale"]

    def mark_synced(self, engine):
        self._cell_of(engine).state = "alive"

    # ---- memory hand-over (colocated) ---------------------------------------------------------------
    def offload(self, tags=("kv_cache", "cuda_graph")):
        with self.lock.hold("offload"):
            for c in self.cells:
                if c.state == "alive":
                    c.engine.pause_generation("retract")
                    c.engine.release_memory_occupation(list(tags))
                    c.state = "offloaded"

    def onload(self, tags=("weights", "kv_cache", "cuda_graph")):
        with self.lock.hold("onload"):
            for c in self.cells:
                if c.state == "offloaded":
                    c.engine.resume_memory_occupation(list(tags))
                    c.engine.continue_generation()
                    c.state = "alive"

    # ---- weight update framing -----------------------------------------------------------------------
    pause_mode = "retract"          # how engines stop for an update (`--pause-generation-mode`: abort | retract | in_place)

    def start_update_weights(self, model: str | None = None) -> list:
        """pause → flush on every engine that follows the trainer; returns those engines."""
        self.lock._lock.acquire()
        self.lock.holder = "update_weights"
        self.updating = True
        targets = self.engines(model)
        for e in targets:
            e.pause_generation(self.pause_mode)
            e.flush_cache()
        return targets

    def end_update_weights(self, version: int, model: str | None = None, ok: bool = True):
        try:
            for e in self.engines(model):
                if ok:
                    e.update_weight_version(version)
                e.continue_generation()
            if ok:
                self.weight_version = version
        finally:
            self.updating = False
            self.lock.holder = None
            self.lock._lock.release()
