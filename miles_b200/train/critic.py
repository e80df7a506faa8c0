"""Value model for PPO: the policy backbone with a scalar head in place of the vocabulary projection.

The reference builds its critic as a Megatron model whose output layer has one column (`--critic-*` flags,
miles/backends/megatron_utils/actor.py role "critic", loss in training_utils/loss/hub/losses.py:422-470).  Here the
head is a replicated fp32 `Linear(hidden, 1)`; values are read at the same rows as policy log-probs (the state
before each response token), so advantages, returns and values share one flat layout.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class ValueHead(nn.Module):
    def __init__(self, hidden: int, device, init_std: float = 0.02, seed: int = 1234):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.weight = nn.Parameter((torch.randn(1, hidden, generator=gen) * init_std).to(device))
        self.bias = nn.Parameter(torch.zeros(1, device=device))

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(h.float(), self.weight, self.bias)


def attach_value_head(model, cfg, dtype, device) -> ValueHead:
    """Add `model.value_head` on the last pipeline stage and drop the language-model head (it receives no gradient
    and would only cost optimizer memory)."""
    model.value_head = ValueHead(cfg.hidden_size, device)
    if getattr(model, "lm_head", None) is not None and not cfg.tie_embeddings:
        model.lm_head.requires_grad_(False)
    return model.value_head
