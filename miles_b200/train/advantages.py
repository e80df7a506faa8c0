"""Advantage / return estimators over a rank's rollout shard.

GRPO / GSPO broadcast the (group-normalised) reward over response tokens; PPO runs chunked GAE on
token rewards −kl_coef·KL_t plus the terminal reward; REINFORCE++ uses discounted returns of the
same token rewards; REINFORCE++-baseline uses reward − kl_coef·KL_t.  Optional DP-wide masked
whitening.  Reference behaviour: miles/backends/training_utils/loss/hub/advantages.py:16-182 and
loss/objective.py:28-126.
"""
from __future__ import annotations

import torch

from . import math_utils as mu


def compute_kl_for_advantages(args, log_probs, ref_log_probs):
    """Per-token KL(π‖π_ref) used inside token rewards; zeros when kl_coef == 0."""
    if getattr(args, "kl_coef", 0.0) == 0 or ref_log_probs is None:
        return torch.zeros_like(log_probs, dtype=torch.float32)
    return mu.compute_approx_kl(log_probs, ref_log_probs, getattr(args, "kl_loss_type", "k1"))


def last_trainable_index(loss_mask: torch.Tensor, seq_ids: torch.Tensor, num_seqs: int):
    """Flat index of the last token with loss_mask > 0 of every sequence, and which sequences have one.  The terminal
    reward is credited there (a response may end in masked tokens: tool or environment output of a multi-turn rollout),
    as in the reference (loss/hub/math_utils.py get_reinforce_plus_plus_returns, get_advantages_and_returns_batch)."""
    R = loss_mask.numel()
    idx = torch.arange(R, device=loss_mask.device)
    cand = torch.where(loss_mask > 0, idx, torch.full_like(idx, -1))
    last = torch.full((num_seqs,), -1, dtype=idx.dtype, device=loss_mask.device)
    last = last.scatter_reduce(0, seq_ids, cand, reduce="amax", include_self=True)
    has = last >= 0
    return last.clamp_min(0), has


def compute_advantages_and_returns(args, *, rewards: torch.Tensor, response_lengths: list[int],
                                   loss_mask: torch.Tensor, log_probs: torch.Tensor | None = None,
                                   ref_log_probs: torch.Tensor | None = None,
                                   values: torch.Tensor | None = None, dp_group=None,
                                   teacher_log_probs: torch.Tensor | None = None,
                                   opd_reverse_kl: torch.Tensor | None = None):
    """rewards [S]; flat tensors [R]. Returns (advantages [R], returns [R])."""
    device = loss_mask.device
    S = len(response_lengths)
    seq_ids = mu.lengths_to_seq_ids(response_lengths, device)
    est = args.advantage_estimator
    r_tok = rewards.float().to(device)[seq_ids]
    if log_probs is None:
        kl = torch.zeros_like(loss_mask, dtype=torch.float32)
    else:
        kl = compute_kl_for_advantages(args, log_probs, ref_log_probs)
    kl_coef = getattr(args, "kl_coef", 0.0)

    if est in ("grpo", "gspo"):
        adv = r_tok.clone()
        ret = adv.clone()
    elif est == "ppo":
        assert values is not None, "PPO needs critic values"
        last, has = last_trainable_index(loss_mask, seq_ids, S)
        tok_r = -kl_coef * kl
        tok_r = tok_r.index_add(0, last[has], rewards.float().to(device)[has])
        adv, ret = mu.masked_gae(tok_r, values.float(), loss_mask, response_lengths, args.gamma, args.lambd)
    elif est == "reinforce_plus_plus":
        last, has = last_trainable_index(loss_mask, seq_ids, S)
        tok_r = -kl_coef * kl
        tok_r = tok_r.index_add(0, last[has], rewards.float().to(device)[has])
        ret = mu.discounted_returns(tok_r, response_lengths, args.gamma)
        # a fully masked sequence has no trainable token to carry the reward: it contributes nothing
        ret = ret * has[seq_ids]
        adv = ret.clone()
    elif est == "reinforce_plus_plus_baseline":
        adv = r_tok - kl_coef * kl
        ret = adv.clone()
    else:
        raise ValueError(f"unknown --advantage-estimator {est}")

    # on-policy distillation: subtract the token-level reverse KL to the teacher
    opd_coef = getattr(args, "opd_kl_coef", 0.0)
    if opd_coef:
        if opd_reverse_kl is not None:
            adv = adv - opd_coef * opd_reverse_kl.float()
        elif teacher_log_probs is not None and log_probs is not None:
            adv = adv - opd_coef * (log_probs.float() - teacher_log_probs.float())

    if getattr(args, "normalize_advantages", False):
        adv = mu.masked_whiten(adv, loss_mask, group=dp_group)
    adv = adv * (loss_mask > 0)
    return adv, ret


def normalize_group_rewards(args, rewards: torch.Tensor, group_sizes: list[int]) -> torch.Tensor:
    """Rollout-side reward post-processing: subtract the prompt-group mean and (GRPO/GSPO, group > 1,
    std > 0) divide by the unbiased std + 1e-6
    (reference: miles/ray/rollout/train_data_conversion.py:275-339)."""
    est = args.advantage_estimator
    if est not in ("grpo", "gspo", "reinforce_plus_plus_baseline") or not getattr(args, "rewards_normalization", True):
        return rewards.float()
    out = rewards.float().clone()
    off = 0
    for n in group_sizes:
        g = out[off:off + n]
        g = g - g.mean()
        if getattr(args, "grpo_std_normalization", True) and est in ("grpo", "gspo") and n > 1:
            std = g.std()
            if std > 0:
                g = g / (std + 1e-6)
        out[off:off + n] = g
        off += n
    return out
