"""Rollout → trainer data contract.

`Sample` carries one generated trajectory from the rollout engine to the trainer.  The field
set follows the reference's record (miles/utils/types.py:67-175) so user hooks written against
it (custom generate / reward / filter functions) keep working; the implementation is ours.

Token-in-token-out: `tokens` holds prompt ids followed by response ids exactly as the engine
produced them, and `rollout_log_probs` / `rollout_routed_experts` are aligned to the response.
"""
from __future__ import annotations

import base64
import copy
import enum
from dataclasses import dataclass, field, fields
from typing import Any

import numpy as np


class Status(enum.Enum):
    PENDING = "pending"
    COMPLETED = "completed"
    TRUNCATED = "truncated"
    ABORTED = "aborted"
    FAILED = "failed"


@dataclass
class RewardSpec:
    """How a single sample is scored (overrides the run-wide --rm-type)."""

    rm_type: str | None = None
    custom_rm_path: str | None = None


@dataclass
class WeightVersionSpan:
    """Weight version that produced `num_tokens` consecutive response tokens."""

    version: int
    num_tokens: int


@dataclass
class SpecInfo:
    """Speculative-decoding counters accumulated over engine calls."""

    spec_num_correct_drafts: int = 0
    spec_num_proposed_drafts: int = 0
    spec_verify_ct: int = 0
    completion_tokens: int = 0

    @property
    def spec_accept_rate(self) -> float:
        p = self.spec_num_proposed_drafts
        return self.spec_num_correct_drafts / p if p else 0.0

    @property
    def spec_accept_length(self) -> float:
        return self.completion_tokens / self.spec_verify_ct if self.spec_verify_ct > 0 else 0.0

    def add(self, meta: dict) -> None:
        ct = meta.get("spec_verify_ct") or 0
        if ct <= 0:
            return
        self.spec_num_correct_drafts += meta.get("spec_num_correct_drafts", 0)
        self.spec_num_proposed_drafts += meta.get("spec_num_proposed_drafts", 0)
        self.spec_verify_ct += ct
        self.completion_tokens += meta.get("completion_tokens", 0)


@dataclass
class PrefixCacheInfo:
    cached_tokens: int = 0
    total_prompt_tokens: int = 0

    @property
    def hit_rate(self) -> float:
        return self.cached_tokens / self.total_prompt_tokens if self.total_prompt_tokens else 0.0

    def add(self, meta: dict) -> None:
        self.cached_tokens += meta.get("cached_tokens", 0)
        self.total_prompt_tokens += meta.get("prompt_tokens", 0)


@dataclass
class Sample:
    group_index: int | None = None
    index: int | None = None
    rollout_id: int | None = None
    prompt: str | list[dict[str, str]] = ""
    tokens: list[int] = field(default_factory=list)
    multimodal_inputs: dict[str, Any] | None = None
    multimodal_train_inputs: dict[str, Any] | None = None
    response: str = ""
    response_length: int = 0
    label: str | None = None
    reward: float | dict[str, Any] | None = None
    loss_mask: list[int] | None = None
    weight_versions: list[WeightVersionSpan] = field(default_factory=list)
    rollout_log_probs: list[float] | None = None
    rollout_topk_token_ids: np.ndarray | None = None
    rollout_topk_log_probs: np.ndarray | None = None
    rollout_sampling_mask: Any | None = None
    rollout_routed_experts: np.ndarray | None = None  # int32 [num_tokens-1, layers, topk]
    rollout_indexer_topk: np.ndarray | None = None
    remove_sample: bool = False
    teacher_log_probs: list[float] | None = None
    opd_reverse_kl: list[float] | None = None
    status: Status = Status.PENDING
    metadata: dict = field(default_factory=dict)
    generate_function_path: str | None = None
    train_metadata: dict | None = None
    reward_spec: RewardSpec | None = None
    routing_key: str | None = None
    trainer_model_id: str | None = None
    non_generation_time: float = 0.0
    spec_info: SpecInfo = field(default_factory=SpecInfo)
    prefix_cache_info: PrefixCacheInfo = field(default_factory=PrefixCacheInfo)

    Status = Status  # `Sample.Status.COMPLETED` spelling used by user hooks

    # ---- derived -------------------------------------------------------------------------
    @property
    def prompt_length(self) -> int:
        return len(self.tokens) - self.response_length

    @property
    def effective_response_length(self) -> int:
        return sum(self.loss_mask) if self.loss_mask is not None else self.response_length

    def get_reward_value(self, reward_key: str | None = None) -> float:
        if isinstance(self.reward, dict):
            if reward_key is None:
                raise ValueError("reward is a dict; pass --reward-key")
            return float(self.reward[reward_key])
        return float(self.reward)

    @property
    def oldest_weight_version(self) -> int | None:
        return min((s.version for s in self.weight_versions), default=None)

    # ---- engine response → sample --------------------------------------------------------
    def append_response(
        self,
        token_ids: list[int],
        log_probs: list[float] | None,
        *,
        text: str = "",
        trainable: bool = True,
    ) -> None:
        """Extend the trajectory with ids produced by the engine (or tool output if not trainable)."""
        n = len(token_ids)
        self.tokens = list(self.tokens) + list(token_ids)
        self.response_length += n
        self.response += text
        if self.loss_mask is None:
            self.loss_mask = [1] * (self.response_length - n)
        self.loss_mask = self.loss_mask + [1 if trainable else 0] * n
        if log_probs is not None:
            if self.rollout_log_probs is None:
                self.rollout_log_probs = [0.0] * (self.response_length - n)
            self.rollout_log_probs = self.rollout_log_probs + [float(x) for x in log_probs]
        elif self.rollout_log_probs is not None:
            self.rollout_log_probs = self.rollout_log_probs + [0.0] * n

    def update_from_meta_info(self, meta: dict, num_new_tokens: int = 0) -> None:
        """Apply finish reason / weight version / spec counters from an engine reply."""
        fr = meta.get("finish_reason") or {}
        kind = fr.get("type") if isinstance(fr, dict) else fr
        if kind == "length":
            self.status = Status.TRUNCATED
        elif kind == "abort":
            self.status = Status.ABORTED
        elif kind in ("stop", "eos"):
            self.status = Status.COMPLETED
        wv = meta.get("weight_version")
        if wv is not None:
            wv = int(wv)
            if self.weight_versions and self.weight_versions[-1].version == wv:
                self.weight_versions[-1].num_tokens += num_new_tokens
            else:
                self.weight_versions.append(WeightVersionSpan(wv, num_new_tokens))
        self.spec_info.add(meta)
        self.prefix_cache_info.add(meta)

    # ---- (de)serialisation ---------------------------------------------------------------
    def to_dict(self) -> dict:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, Status):
                v = v.value
            elif isinstance(v, np.ndarray):
                v = {"__nd__": base64.b64encode(np.ascontiguousarray(v).tobytes()).decode(),
                     "dtype": str(v.dtype), "shape": list(v.shape)}
            elif isinstance(v, (SpecInfo, PrefixCacheInfo, RewardSpec)):
                v = dict(v.__dict__)
            elif f.name == "weight_versions":
                v = [[s.version, s.num_tokens] for s in v]
            out[f.name] = v
        return out

    @staticmethod
    def from_dict(d: dict) -> "Sample":
        d = dict(d)
        kw: dict[str, Any] = {}
        names = {f.name for f in fields(Sample)}
        for k, v in d.items():
            if k not in names:
                continue
            if k == "status":
                v = Status(v)
            elif isinstance(v, dict) and "__nd__" in v:
                v = np.frombuffer(base64.b64decode(v["__nd__"]), dtype=v["dtype"]).reshape(v["shape"]).copy()
            elif k == "spec_info":
                v = SpecInfo(**v)
            elif k == "prefix_cache_info":
                v = PrefixCacheInfo(**v)
            elif k == "reward_spec" and v is not None:
                v = RewardSpec(**v)
            elif k == "weight_versions":
                v = [WeightVersionSpan(a, b) for a, b in v]
            kw[k] = v
        return Sample(**kw)

    def clone(self) -> "Sample":
        return copy.deepcopy(self)


def decode_routed_experts(b64, num_tokens: int, num_layers: int, topk: int) -> np.ndarray:
    """Engine replies carry routed experts as base64 int32 (an engine in this process hands over the array itself);
    shape [num_tokens-1, layers, topk].

    An all-zero buffer means the engine never recorded routing and is rejected
    (reference behaviour: miles/rollout/generate_utils/generate_endpoint_utils.py:142-162).
    """
    if isinstance(b64, np.ndarray):
        arr = np.ascontiguousarray(b64, dtype=np.int32).reshape(num_tokens - 1, num_layers, topk)
    else:
        arr = np.frombuffer(base64.b64decode(b64), dtype=np.int32).reshape(num_tokens - 1, num_layers, topk).copy()
    if arr.size and not arr.any():
        raise ValueError("routed_experts buffer is all zero: engine did not record routing")
    return arr


def encode_routed_experts(arr: np.ndarray) -> str:
    return base64.b64encode(np.ascontiguousarray(arr, dtype=np.int32).tobytes()).decode()


@dataclass
class RolloutDataPack:
    """Handle returned by the rollout executor: which samples and where their tensors live."""

    rollout_id: int
    sample_indices: list[int]
    data_ref: Any  # object-store keys, one per DP rank
    metrics: dict = field(default_factory=dict)
