"""Training metrics: reduction over data-parallel ranks, throughput / MFU, rollout-data statistics and CI gates.

Reference: miles/backends/training_utils/metrics/log_utils.py:33-556 (gather/reduce of log dicts, rollout-data stats),
metrics/perf.py:14-64 (`perf/*_time`, TFLOPs, MFU, tokens/s) and metrics/checks.py (KL == 0 at step 0, grad-norm
record/replay for determinism checks).
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

PEAK_BF16_TFLOPS = {"B200": 2250.0, "GB200": 2500.0, "H100": 989.0, "H200": 989.0, "A100": 312.0}   # dense, per GPU


def device_peak_tflops(name: str | None = None) -> float:
    """Datasheet dense bf16 peak (the reference's MFU denominator, miles/utils/device_flops.py:6-16)."""
    if name is None and torch.cuda.is_available():
        name = torch.cuda.get_device_name(0)
    for k, v in PEAK_BF16_TFLOPS.items():
        if name and k in name:
            return v
    return PEAK_BF16_TFLOPS["B200"]


def reduce_log_dict(sums: dict[str, float], counts: dict[str, float] | float, group=None) -> dict[str, float]:
    """Weighted mean of every metric over the group: Σ_rank sum / Σ_rank count, one all-reduce of a packed vector.
    Keys missing on some ranks are handled by exchanging the key set first."""
    keys = sorted(sums)
    world = dist.get_world_size(group) if dist.is_initialized() and group is not None else 1
    if world > 1:
        all_keys: list = [None] * world
        dist.all_gather_object(all_keys, keys, group=group)
        keys = sorted(set().union(*all_keys))
    cnt = (lambda k: counts.get(k, 0.0)) if isinstance(counts, dict) else (lambda k: float(counts) if k in sums else 0.0)
    vec = torch.tensor([sums.get(k, 0.0) for k in keys] + [cnt(k) for k in keys], dtype=torch.float64)
    if world > 1:
        dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
        vec = vec.to(dev)
        dist.all_reduce(vec, group=group)
        vec = vec.cpu()
    n = len(keys)
    return {k: float(vec[i] / vec[n + i]) if vec[n + i] > 0 else 0.0 for i, k in enumerate(keys)}


def perf_metrics(cfg, num_tokens: int, seq_len_mean: float, seconds: float, n_gpus: int = 1, prefix: str = "actor_train",
                 forward_only: bool = False, peak_tflops: float | None = None) -> dict[str, float]:
    """tokens/s, model TFLOP/s per GPU and MFU for a phase that processed `num_tokens` tokens in `seconds`."""
    flops_tok = cfg.flops_per_token(int(seq_len_mean))
    if forward_only:
        flops_tok /= 3.0
    tflops = flops_tok * num_tokens / max(seconds, 1e-9) / 1e12 / max(1, n_gpus)
    peak = peak_tflops or device_peak_tflops()
    return {f"perf/{prefix}_time": seconds, f"perf/{prefix}_tok_per_s": num_tokens / max(seconds, 1e-9),
            f"perf/{prefix}_tflops": tflops, f"perf/{prefix}_mfu": tflops / peak}


def rollout_data_stats(shard: dict) -> dict[str, float]:
    """Statistics of a train-data shard before training (reference: log_rollout_data)."""
    resp = shard["response_lengths"]
    n = max(1, len(resp))
    out = {"rollout/response_len/mean": sum(resp) / n, "rollout/response_len/max": float(max(resp, default=0)),
           "rollout/total_len/mean": sum(shard["total_lengths"]) / n, "rollout/rewards/mean": sum(shard["rewards"]) / n}
    if "raw_reward" in shard:
        out["rollout/raw_reward/mean"] = sum(shard["raw_reward"]) / max(1, len(shard["raw_reward"]))
    if "truncated" in shard:
        out["rollout/truncated_ratio"] = sum(shard["truncated"]) / n
    masks = shard.get("loss_masks")
    if masks:
        tot = sum(len(m) for m in masks)
        out["rollout/loss_mask_ratio"] = sum(sum(m) for m in masks) / max(1, tot)
    if "weight_versions" in shard:
        vs = [v for v in shard["weight_versions"] if v is not None]
        if vs:
            out["rollout/weight_version/min"], out["rollout/weight_version/max"] = float(min(vs)), float(max(vs))
    return out


# ---- CI gates ------------------------------------------------------------------------------------------------

def check_kl_zero_at_step0(log_probs: torch.Tensor, ref_log_probs: torch.Tensor, tol: float = 1e-5):
    d = (log_probs.float() - ref_log_probs.float()).abs().max().item() if log_probs.numel() else 0.0
    assert d < tol, f"KL between actor and reference must be 0 before the first update, max |Δlogp| = {d}"


class GradNormRecorder:
    """Record grad norms per step to a file, or replay the file and require equality (determinism / resume checks)."""

    def __init__(self, path: str, mode: str = "record", rtol: float = 0.0):
        assert mode in ("record", "replay")
        self.path, self.mode, self.rtol = path, mode, rtol
        self.values: dict[str, float] = {}
        if mode == "replay":
            with open(path) as f:
                self.values = json.load(f)

    def step(self, step_id: int, grad_norm: float):
        key = str(step_id)
        if self.mode == "record":
            self.values[key] = float(grad_norm)
            os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
            with open(self.path, "w") as f:
                json.dump(self.values, f)
            return
        assert key in self.values, f"no recorded grad norm for step {step_id}"
        want = self.values[key]
        assert abs(grad_norm - want) <= self.rtol * abs(want), f"step {step_id}: grad norm {grad_norm} != recorded {want}"
