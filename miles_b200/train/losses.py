"""Loss hub: policy (PPO-clip / dual-clip / GSPO / OPSM / TIS / entropy / KL), value, SFT and custom.

The inputs are flat response-token tensors (`LossBatch`); reduction is "sum over samples of the
per-sample masked mean" by default or a plain token sum with `--calculate-per-token-loss`
(reference semantics: miles/backends/training_utils/loss/hub/losses.py:64-404 and
loss/objective.py:128-229).  Metric keys match the reference so dashboards keep working.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..utils.misc import load_function
from . import math_utils as mu


@dataclass
class LossBatch:
    """Flat per-response-token view of one micro-batch (R tokens, S samples)."""

    response_lengths: list[int]
    loss_mask: torch.Tensor                       # [R] float {0,1}
    seq_ids: torch.Tensor                         # [R] long
    advantages: torch.Tensor | None = None        # [R]
    returns: torch.Tensor | None = None           # [R]
    old_log_probs: torch.Tensor | None = None     # [R] trainer-recomputed (or rollout's)
    ref_log_probs: torch.Tensor | None = None     # [R]
    rollout_log_probs: torch.Tensor | None = None  # [R] from the engine
    old_values: torch.Tensor | None = None        # [R]
    denominators: torch.Tensor | None = None      # [S] overrides per-sample mask sums (rollout_mask_sums)
    loss_weights: torch.Tensor | None = None      # [S]
    extra: dict = field(default_factory=dict)

    @property
    def num_samples(self) -> int:
        return len(self.response_lengths)

    def reducer(self, per_token: bool, mask: torch.Tensor | None = None) -> Callable[[torch.Tensor], torch.Tensor]:
        m = self.loss_mask if mask is None else mask
        if per_token:
            return lambda x: (x * m).sum()
        den = self.denominators
        if den is None:
            den = mu.segment_sum(self.loss_mask, self.seq_ids, self.num_samples)
        w = 1.0 / den.float().clamp_min(1.0)
        if self.loss_weights is not None:
            w = w * self.loss_weights.float()
        tok_w = w[self.seq_ids]
        return lambda x: (x * m * tok_w).sum()


# ---- importance-sampling corrections -----------------------------------------------------------

def vanilla_tis(args, pg_loss, train_log_probs, rollout_log_probs, loss_mask):
    """Truncated importance sampling between the trainer's and the engine's view of the old policy."""
    ratio = torch.exp((train_log_probs.float() - rollout_log_probs.float()).clamp(-20, 20))
    lo = getattr(args, "tis_clip_low", 0.0) or 0.0
    hi = args.tis_clip
    w = ratio.clamp(min=lo, max=hi).detach()
    metrics = {
        "tis": w,
        "tis_clipfrac": ((ratio > hi) | (ratio < lo)).float(),
        "tis_abs": (ratio - 1.0).abs(),
    }
    return pg_loss * w, loss_mask, metrics


def icepop_tis(args, pg_loss, train_log_probs, rollout_log_probs, loss_mask):
    """IcePop: tokens whose ratio leaves [low, high] contribute nothing (masked, not clipped)."""
    ratio = torch.exp((train_log_probs.float() - rollout_log_probs.float()).clamp(-20, 20))
    lo = getattr(args, "tis_clip_low", 0.0) or 0.0
    hi = args.tis_clip
    inside = ((ratio >= lo) & (ratio <= hi)).float()
    w = (ratio * inside).detach()
    return pg_loss * w, loss_mask, {"tis": w, "tis_clipfrac": 1.0 - inside, "tis_abs": (ratio - 1.0).abs()}


# ---- policy loss --------------------------------------------------------------------------------

def policy_loss_function(args, batch: LossBatch, log_probs: torch.Tensor, entropy: torch.Tensor | None):
    """Returns (loss scalar, metrics dict of scalars already reduced with the batch reducer)."""
    per_token = getattr(args, "calculate_per_token_loss", False)
    S = batch.num_samples
    mask = batch.loss_mask
    red = batch.reducer(per_token)
    log_probs = log_probs.float()

    if getattr(args, "use_rollout_logprobs", False):
        old = batch.rollout_log_probs
    else:
        old = batch.old_log_probs
    if old is None:  # skipped the forward-only pass: strictly on-policy
        old = log_probs.detach()
    old = old.float()

    active = mask > 0
    adv = torch.where(active, torch.nan_to_num(batch.advantages.float(), nan=0.0, posinf=0.0, neginf=0.0),
                      torch.zeros((), device=mask.device))
    if args.advantage_estimator == "gspo":
        ppo_kl = mu.compute_gspo_kl(log_probs, old, mask, batch.seq_ids, S)
    else:
        ppo_kl = old - log_probs
    ppo_kl = torch.where(active, torch.nan_to_num(ppo_kl, nan=0.0, posinf=0.0, neginf=0.0),
                         torch.zeros((), device=mask.device))

    pg_loss, pg_clipfrac = mu.compute_policy_loss(ppo_kl, adv, args.eps_clip, args.eps_clip_high,
                                                  getattr(args, "eps_clip_c", None))
    metrics: dict[str, torch.Tensor] = {}
    if getattr(args, "use_opsm", False):
        keep, frac = mu.compute_opsm_mask(log_probs, old, adv, mask, batch.seq_ids, S, args.opsm_delta)
        pg_loss = pg_loss * keep
        metrics["opsm_clipfrac"] = frac * (S if not per_token else mask.sum())

    pg_red = red
    tis_metrics: dict[str, torch.Tensor] = {}
    if getattr(args, "use_tis", False) or getattr(args, "get_mismatch_metrics", False):
        assert batch.rollout_log_probs is not None, "TIS needs rollout_log_probs from the engine"
        train_old = batch.old_log_probs if batch.old_log_probs is not None else log_probs.detach()
        if getattr(args, "custom_tis_function_path", None):
            tis_fn = load_function(args.custom_tis_function_path)
        else:
            tis_fn = icepop_tis if getattr(args, "tis_mode", "clip") == "icepop" else vanilla_tis
        new_loss, new_mask, tis_metrics = tis_fn(args, pg_loss, train_old, batch.rollout_log_probs, mask)
        tis_metrics = dict(tis_metrics)
        tis_metrics["ois"] = torch.exp(-ppo_kl)
        if getattr(args, "use_tis", False):
            pg_loss = new_loss
            pg_red = batch.reducer(per_token, new_mask)

    loss_pg = pg_red(pg_loss)
    metrics["pg_loss"] = loss_pg.detach()
    metrics["pg_clipfrac"] = red(pg_clipfrac)
    metrics["ppo_kl"] = red(ppo_kl.detach())
    for k, v in tis_metrics.items():
        metrics[k] = red(v.detach().float())

    # effective-sample-size ratio of the per-token IS weights w = exp(−ppo_kl): (Σw)² / (n Σw²) per sample
    w = torch.exp(-ppo_kl.detach()) * mask
    sw = mu.segment_sum(w, batch.seq_ids, S)
    sw2 = mu.segment_sum(w * w, batch.seq_ids, S)
    n = mu.segment_sum(mask, batch.seq_ids, S)
    ess = (sw * sw / (n * sw2).clamp_min(1e-12))
    metrics["ess_ratio"] = (ess * n).sum() if per_token else torch.where(n > 0, ess, torch.zeros_like(ess)).sum()

    loss = loss_pg
    if entropy is not None:
        ent = red(entropy.float())
        metrics["entropy_loss"] = ent.detach()
        if getattr(args, "entropy_coef", 0.0):
            loss = loss - args.entropy_coef * ent
    if getattr(args, "use_kl_loss", False):
        assert batch.ref_log_probs is not None, "--use-kl-loss needs reference log-probs"
        ratio = None
        if getattr(args, "use_unbiased_kl", False):
            ratio = torch.exp((log_probs - old).clamp(-20, 20))     # live: its gradient is part of the estimator
        kl = mu.compute_approx_kl(log_probs, batch.ref_log_probs, args.kl_loss_type, ratio)
        kl_loss = red(kl)
        metrics["kl_loss"] = kl_loss.detach()
        loss = loss + args.kl_loss_coef * kl_loss
    if batch.rollout_log_probs is not None:
        base = batch.old_log_probs if batch.old_log_probs is not None else log_probs.detach()
        diff = base.float() - batch.rollout_log_probs.float()
        metrics["train_rollout_logprob_abs_diff"] = red(diff.abs())
        metrics["train_rollout_kl"] = red(mu.compute_approx_kl(batch.rollout_log_probs, base, "k3"))
    metrics["loss"] = loss.detach()
    return loss, metrics


def value_loss_function(args, batch: LossBatch, values: torch.Tensor, _entropy=None):
    """Clipped value regression toward GAE returns."""
    red = batch.reducer(getattr(args, "calculate_per_token_loss", False))
    v = values.float()
    old_v = batch.old_values.float() if batch.old_values is not None else v.detach()
    clip = getattr(args, "value_clip", 0.2)
    v_clipped = old_v + (v - old_v).clamp(-clip, clip)
    ret = batch.returns.float()
    l1, l2 = (v - ret) ** 2, (v_clipped - ret) ** 2
    loss = 0.5 * red(torch.maximum(l1, l2))
    return loss, {"value_loss": loss.detach(), "value_clipfrac": red((l2 > l1).float()), "loss": loss.detach()}


def sft_loss_function(args, batch: LossBatch, log_probs: torch.Tensor, _entropy=None):
    red = batch.reducer(getattr(args, "calculate_per_token_loss", False))
    loss = -red(log_probs.float())
    return loss, {"sft_loss": loss.detach(), "loss": loss.detach()}


# ---- Tinker-style losses -------------------------------------------------------------------------

def _tinker_cross_entropy(args, batch, log_probs, _e=None):
    w = batch.extra.get("weights", batch.loss_mask)
    loss = -(log_probs.float() * w).sum()
    return loss, {"loss": loss.detach()}


def _tinker_importance_sampling(args, batch, log_probs, _e=None):
    old = batch.rollout_log_probs.float()
    ratio = torch.exp((log_probs.float() - old).clamp(-20, 20))
    loss = -(ratio * batch.advantages.float() * batch.loss_mask).sum()
    return loss, {"loss": loss.detach()}


def _tinker_ppo(args, batch, log_probs, _e=None):
    cfg = batch.extra.get("loss_fn_config") or {}
    lo, hi = cfg.get("clip_low_threshold", 0.8), cfg.get("clip_high_threshold", 1.2)
    ratio = torch.exp((log_probs.float() - batch.rollout_log_probs.float()).clamp(-20, 20))
    a = batch.advantages.float()
    loss = -(torch.minimum(ratio * a, ratio.clamp(lo, hi) * a) * batch.loss_mask).sum()
    return loss, {"loss": loss.detach()}


def _tinker_cispo(args, batch, log_probs, _e=None):
    cfg = batch.extra.get("loss_fn_config") or {}
    lo, hi = cfg.get("clip_low_threshold", 0.8), cfg.get("clip_high_threshold", 1.2)
    ratio = torch.exp((log_probs.float() - batch.rollout_log_probs.float()).clamp(-20, 20))
    loss = -(ratio.clamp(lo, hi).detach() * batch.advantages.float() * log_probs.float() * batch.loss_mask).sum()
    return loss, {"loss": loss.detach()}


def _tinker_dro(args, batch, log_probs, _e=None):
    cfg = batch.extra.get("loss_fn_config") or {}
    beta = cfg.get("beta", 0.05)
    d = log_probs.float() - batch.rollout_log_probs.float()
    loss = -((d * batch.advantages.float() - 0.5 * beta * d * d) * batch.loss_mask).sum()
    return loss, {"loss": loss.detach()}


TINKER_LOSSES = {
    "cross_entropy": _tinker_cross_entropy,
    "importance_sampling": _tinker_importance_sampling,
    "ppo": _tinker_ppo,
    "cispo": _tinker_cispo,
    "dro": _tinker_dro,
}


def get_loss_function(args, loss_fn_name: str | None = None):
    if loss_fn_name is not None:
        return TINKER_LOSSES[loss_fn_name]
    lt = getattr(args, "loss_type", "policy_loss")
    if lt == "policy_loss":
        return policy_loss_function
    if lt == "value_loss":
        return value_loss_function
    if lt == "sft_loss":
        return sft_loss_function
    if lt == "custom_loss":
        return load_function(args.custom_loss_function_path)
    raise ValueError(f"unknown --loss-type {lt}")


def loss_function(args, batch: LossBatch, log_probs, entropy, *, global_batch_size: int,
                  global_num_tokens: torch.Tensor | float | None = None, loss_fn_name: str | None = None):
    """Loss scaled for gradient accumulation under a SUM gradient reduction over data-parallel ranks.

    Sample-mean mode: Σ_samples mean_tokens(·) / global_batch_size, so that summing over micro-batches
    and DP ranks gives the mean over the global batch.  Per-token mode: Σ_tokens(·) / global token
    count of the optimizer step (the trainer all-reduces the count once per step).  The reference
    reaches the same value through Megatron's averaging conventions
    (miles/backends/training_utils/loss/objective.py:197-215).
    Returns (scaled loss, {metric: reduced value}, count) where count weights the metric averages.
    """
    fn = get_loss_function(args, loss_fn_name)
    loss, metrics = fn(args, batch, log_probs, entropy)
    if getattr(args, "calculate_per_token_loss", False):
        count = batch.loss_mask.sum()
        denom = global_num_tokens if global_num_tokens is not None else count.clamp_min(1.0)
        scaled = loss / denom
    else:
        count = torch.tensor(float(batch.num_samples), device=loss.device)
        scaled = loss / float(global_batch_size)
    return scaled, metrics, count
