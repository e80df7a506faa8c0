"""Routing replay (R3): make the trainer's MoE layers route tokens exactly as the rollout engine did.

The reference wraps each router's top-k function in a `BaseReplayManager` with stages
`fallthrough / record / replay_forward / replay_backward` (miles/utils/replay_base.py:14-241) and feeds it
`[tokens-1, layers, topk]` index tensors re-sliced per micro-batch (replay/data.py:30-140).  In this package the model
takes recorded indices through `ForwardMeta.replay_topk` (`models/qwen3.py`, packed by
`train.data.pack_micro_batch(with_replay=True)`); this module provides the same manager object for custom models and
plugins whose routers are plain callables: wrap the top-k function once, switch stages around forward passes.

Semantics kept from the reference: in replay stages the *indices* come from the record, the *weights* are re-gathered
from the current scores (`scores.gather(1, idx)`, optionally renormalised) so the gate still receives gradient; rows
recorded as all −1 (padding, or tokens the engine never routed) fall through to the live top-k.
"""
from __future__ import annotations

from collections import deque
from typing import Callable

import torch

STAGES = ("fallthrough", "record", "replay_forward", "replay_backward")


class ReplayManager:
    def __init__(self, normalize: bool = True):
        self.stage = "fallthrough"
        self.normalize = normalize
        self.recorded: list[torch.Tensor] = []          # record stage: one [T, k] per router call, in call order
        self._fwd: deque[torch.Tensor] = deque()        # replay queues (forward order; backward = recompute order)
        self._bwd: deque[torch.Tensor] = deque()

    # ---- stage control ---------------------------------------------------------------------------
    def set_stage(self, stage: str):
        assert stage in STAGES, stage
        self.stage = stage

    def clear(self):
        self.recorded.clear()
        self._fwd.clear()
        self._bwd.clear()

    def load(self, per_layer_indices: list[torch.Tensor]):
        """Indices to replay, one [T, k] tensor per router call of one forward pass."""
        self._fwd = deque(per_layer_indices)
        # activation recomputation calls the routers again during backward, in the same order per recomputed layer
        self._bwd = deque(per_layer_indices)

    def load_packed(self, replay_topk: torch.Tensor):
        """[T, L_moe, k] (the layout `pack_micro_batch` produces) → per-layer queue."""
        self.load([replay_topk[:, l, :] for l in range(replay_topk.shape[1])])

    # ---- the wrapper -------------------------------------------------------------------------------
    def wrap(self, topk_fn: Callable[[torch.Tensor, int], tuple[torch.Tensor, torch.Tensor]]):
        """topk_fn(scores [T, E], k) → (weights [T, k], indices [T, k]); returns a function with the same signature."""

        def routed(scores: torch.Tensor, k: int):
            if self.stage == "fallthrough":
                return topk_fn(scores, k)
            if self.stage == "record":
                w, idx = topk_fn(scores, k)
                self.recorded.append(idx.detach().to(torch.int32).cpu())
                return w, idx
            q = self._fwd if self.stage == "replay_forward" else self._bwd
            assert q, f"no recorded routing left for stage {self.stage}"
            idx = q.popleft().to(scores.device).long()
            assert idx.shape[0] == scores.shape[0], f"recorded {idx.shape[0]} tokens, router saw {scores.shape[0]}"
            bad = (idx < 0).all(dim=-1)
            if bad.any():
                _, live = topk_fn(scores, k)
                idx = torch.where(bad[:, None], live.long(), idx)
            w = scores.gather(1, idx)
            if self.normalize:
                w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
            return w, idx

        return routed

    def stacked_record(self) -> torch.Tensor:
        """[T, L, k] int32 of everything recorded since `clear()` (what the engine returns as `routed_experts`)."""
        return torch.stack(self.recorded, dim=1)
