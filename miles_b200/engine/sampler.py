"""Token sampling with returned log-probabilities.

The log-prob reported for a sampled token is log-softmax of the temperature-scaled logits *before*
top-p / top-k truncation — the quantity the trainer recomputes, so rollout and train log-probs are
comparable (`train_rollout_logprob_abs_diff`).  On CUDA the no-truncation case is one fused kernel
(max / sum-exp / Gumbel-argmax / log-prob per row); truncation falls back to a sort.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_new_tokens: int = 128
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    no_stop_trim: bool = False
    seed: int | None = None

    @staticmethod
    def from_dict(d: dict | None) -> "SamplingParams":
        d = dict(d or {})
        known = {k: d[k] for k in SamplingParams.__dataclass_fields__ if k in d}
        if "stop_token_ids" in known and known["stop_token_ids"] is None:
            known["stop_token_ids"] = []
        return SamplingParams(**known)


def _draw(probs: torch.Tensor, generator, seeds, step: int) -> torch.Tensor:
    """One categorical draw per row.  With per-row `seeds` (and no shared generator) each row inverts its CDF at a
    uniform number that depends on (seed, step) alone, so a request samples the same tokens whatever it is batched with."""
    if generator is not None or seeds is None:
        return torch.multinomial(probs, 1, generator=generator).squeeze(1)
    u = torch.empty(probs.shape[0], dtype=torch.float64)
    for i, s in enumerate(seeds.tolist()):
        u[i] = torch.rand(1, generator=torch.Generator().manual_seed((int(s) * 2654435761 + step) % (2 ** 63 - 1)),
                          dtype=torch.float64)
    cdf = probs.double().cumsum(-1)
    u = (u.to(probs.device) * cdf[:, -1]).unsqueeze(1)
    return torch.searchsorted(cdf, u).squeeze(1).clamp_(max=probs.shape[1] - 1)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor | None = None,
           top_k: torch.Tensor | None = None, generator: torch.Generator | None = None,
           seeds: torch.Tensor | None = None, step: int = 0):
    """logits fp32 [B,V]; temperature [B] (0 → greedy). Returns (tokens int64 [B], logprobs fp32 [B])."""
    B, V = logits.shape
    greedy = temperature <= 0
    t = torch.where(greedy, torch.ones_like(temperature), temperature).float()
    need_trunc = (top_p is not None and bool((top_p < 1.0).any())) or (top_k is not None and bool((top_k > 0).any()))
    if logits.is_cuda and not need_trunc:
        from .. import ops

        return ops._k().sample_logprob(logits, t, greedy, seeds, step)
    scaled = logits.float() / t[:, None]
    logp = torch.log_softmax(scaled, dim=-1)
    probs = logp.exp()
    if need_trunc:
        sp, si = probs.sort(dim=-1, descending=True)
        keep = torch.ones_like(sp, dtype=torch.bool)
        if top_p is not None:
            cum = sp.cumsum(-1)
            keep &= (cum - sp) < top_p[:, None]
        if top_k is not None:
            k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V))
            keep &= torch.arange(V, device=logits.device)[None, :] < k[:, None]
        sp = sp * keep
        sp = sp / sp.sum(-1, keepdim=True)
        pick = _draw(sp, generator, seeds, step)
        tok = si.gather(1, pick[:, None]).squeeze(1)
    else:
        tok = _draw(probs, generator, seeds, step)
    tok = torch.where(greedy, logits.argmax(-1), tok)
    return tok, logp.gather(1, tok[:, None]).squeeze(1)
