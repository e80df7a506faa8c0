"""Rollout filters (reference: miles/rollout/filter_hub/*, data_source.py:227-231).

* dynamic sampling filters  `fn(args, group) -> bool`   keep a prompt group? (`--dynamic-sampling-filter-path`)
* buffer filters            `fn(args, rollout_id, buffer, n) -> groups`   which buffered partial groups resume first
* per-sample filters        `fn(args, groups) -> None`   mark `remove_sample` on individual samples (`--rollout-sample-filter-path`)
"""
from __future__ import annotations

import statistics

from ..types import Sample, Status


def _reward(args, s: Sample) -> float:
    return s.get_reward_value(getattr(args, "reward_key", None))


# ---- dynamic sampling -------------------------------------------------------------------------------------

def check_reward_nonzero_std(args, group: list[Sample], **kw) -> bool:
    """DAPO dynamic sampling: drop groups whose rewards are all equal (no learning signal under GRPO)."""
    r = [_reward(args, s) for s in group]
    return len(r) > 1 and statistics.pstdev(r) > 0


def check_no_truncated(args, group: list[Sample], **kw) -> bool:
    return all(s.status != Status.TRUNCATED for s in group)


def check_mean_reward_in_range(args, group: list[Sample], **kw) -> bool:
    lo, hi = getattr(args, "dynamic_filter_reward_range", (0.0, 1.0))
    m = sum(_reward(args, s) for s in group) / max(1, len(group))
    return lo < m < hi


# ---- buffer -------------------------------------------------------------------------------------------------

def pop_first(args, rollout_id, buffer: list[list[Sample]], num: int) -> list[list[Sample]]:
    out = buffer[:num]
    del buffer[:num]
    return out


def pop_longest_first(args, rollout_id, buffer: list[list[Sample]], num: int) -> list[list[Sample]]:
    """Resume the partial groups that already hold the most tokens (they finish soonest)."""
    buffer.sort(key=lambda g: -sum(s.response_length for s in g))
    return pop_first(args, rollout_id, buffer, num)


# ---- per-sample ---------------------------------------------------------------------------------------------

def remove_truncated(args, groups: list[list[Sample]]) -> None:
    for g in groups:
        for s in g:
            if s.status == Status.TRUNCATED:
                s.remove_sample = True


def remove_overlong(args, groups: list[list[Sample]]) -> None:
    limit = getattr(args, "rollout_max_response_len", None)
    for g in groups:
        for s in g:
            if limit and s.response_length >= limit:
                s.remove_sample = True
