"""True-on-policy mode: contracts that make trainer and rollout numerics bit-identical.

Reference: miles/true_on_policy/* (contracts + per-model profiles, 522 LoC): when `--true-on-policy-mode` is on, every
source of train/rollout numeric divergence is pinned — same kernels and reduction orders on both sides, fp32 logits,
no sampling-time truncation, deterministic collectives — so `train_rollout_logprob_abs_diff` is exactly 0 and
importance weights are exactly 1.

In this package trainer and engine already share the model code and kernels; what differs by default is listed in
`CONTRACTS`.  `apply(args)` sets the flags that close each gap, `verify(history)` is the CI gate.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class Contract:
    name: str
    why: str
    args: dict            # argparse attributes forced
    env: dict             # environment forced (kernel selection)


CONTRACTS = [
    Contract("same_attention_kernel",
             "prefill uses the tcgen05 forward, training may recompute with the mma.sync forward during backward; decode "
             "uses the paged split-KV kernel whose reduction order differs from the varlen kernel",
             {}, {"MILES_TC_ATTENTION": "1", "MILES_DECODE_SPLITS": "1"}),
    Contract("no_split_k", "split-K GEMMs add K slices in a different order than the single-pass GEMM the trainer runs",
             {}, {"MILES_SPLIT_K": "0"}),
    Contract("fp32_logits", "log-probs must come from fp32 logits on both sides", {"log_probs_fp32": True}, {}),
    Contract("no_truncated_sampling", "top-p / top-k renormalise the distribution the engine samples from",
             {"rollout_top_p": 1.0, "rollout_top_k": -1}, {}),
    Contract("temperature_shared", "the trainer divides logits by the rollout temperature before log-softmax", {}, {}),
    Contract("no_sequence_parallel_mismatch", "reduce-scatter (trainer, SP) and all-reduce (engine) sum in different orders",
             {"sequence_parallel": False}, {}),
    Contract("routing_replay", "MoE ties at the top-k boundary may resolve differently; replay the engine's routing",
             {"use_rollout_routing_replay": True, "use_routing_replay": True}, {}),
    Contract("rollout_logprobs_as_old", "the recomputed old log-probs are redundant once both sides agree bit for bit",
             {"use_rollout_logprobs": False}, {}),
]

MODEL_PROFILES = {
    # which contracts a model family needs (dense models have no router)
    "dense": [c.name for c in CONTRACTS if c.name != "routing_replay"],
    "moe": [c.name for c in CONTRACTS],
}


def apply(args, profile: str | None = None) -> list[str]:
    """Force the flags / environment of the selected contracts.  Returns the names applied."""
    if profile is None:
        profile = "moe" if getattr(args, "num_experts", 0) or "moe" in str(getattr(args, "model_name", "")).lower() \
            or "A3B" in str(getattr(args, "model_name", "")) else "dense"
    names = MODEL_PROFILES[profile]
    for c in CONTRACTS:
        if c.name not in names:
            continue
        for k, v in c.args.items():
            setattr(args, k, v)
        for k, v in c.env.items():
            os.environ[k] = v
    return names


def verify(history_rows: list[dict], tol: float = 0.0) -> None:
    """CI gate: every step's train/rollout log-prob difference is (at most) `tol`; TIS weights, if logged, are 1."""
    for r in history_rows:
        d = r.get("train/train_rollout_logprob_abs_diff")
        if d is not None and d > tol:
            raise AssertionError(f"step {r.get('rollout/step')}: train/rollout log-prob difference {d} > {tol}")
        t = r.get("train/tis")
        if t is not None and abs(t - 1.0) > max(tol, 1e-12):
            raise AssertionError(f"step {r.get('rollout/step')}: importance weight {t} != 1")
