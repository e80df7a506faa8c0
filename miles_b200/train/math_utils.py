"""Token-level RL math on packed response tensors.

All functions take flat tensors over the response tokens of a micro-batch ([R]) plus `seq_ids`
([R], which sample each token belongs to) instead of python lists of per-sample tensors, so that a
micro-batch is a handful of launches regardless of how many samples it packs.

Behaviour follows the reference's loss hub (miles/backends/training_utils/loss/hub/math_utils.py:
138-277 KL estimators and PPO clip, :183-250 OPSM / GSPO sequence KL, :818-958 chunked GAE).
"""
from __future__ import annotations

import torch


# ---- segment helpers ---------------------------------------------------------------------------

def segment_sum(x: torch.Tensor, seq_ids: torch.Tensor, num_seqs: int) -> torch.Tensor:
    out = torch.zeros(num_seqs, dtype=x.dtype, device=x.device)
    return out.index_add(0, seq_ids, x)


def segment_mean_expand(x, mask, seq_ids, num_seqs):
    """Per-sequence masked mean of x, broadcast back to every token of the sequence."""
    s = segment_sum(x * mask, seq_ids, num_seqs)
    n = segment_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
    return (s / n)[seq_ids]


def lengths_to_seq_ids(lengths, device) -> torch.Tensor:
    lens = torch.as_tensor(lengths, device=device, dtype=torch.long)
    return torch.repeat_interleave(torch.arange(len(lengths), device=device), lens)


# ---- KL estimators -----------------------------------------------------------------------------

def compute_approx_kl(log_probs, log_probs_base, kl_loss_type: str = "k1", importance_ratio=None):
    """Schulman's estimators with d = logp − logp_base: k1 d; k2 d²/2; k3 exp(−d) − 1 + d;
    low_var_kl = k3 with a guarded exponent, clamped to [−10, 10] AFTER the optional × importance ratio
    (reference: loss/hub/math_utils.py:139-180)."""
    d = log_probs.float() - log_probs_base.float()
    if kl_loss_type == "k1":
        kl = d
    elif kl_loss_type == "k2":
        kl = 0.5 * d * d
    elif kl_loss_type == "k3":
        kl = torch.exp(-d) - 1.0 + d
    elif kl_loss_type == "low_var_kl":
        nd = torch.clamp(torch.nan_to_num(-d, nan=0.0, posinf=20.0, neginf=-20.0), min=-20.0, max=20.0)
        kl = torch.exp(nd) - 1.0 - nd
    else:
        raise ValueError(f"unknown kl_loss_type {kl_loss_type}")
    if importance_ratio is not None:
        kl = kl * importance_ratio
    if kl_loss_type == "low_var_kl":
        kl = torch.clamp(kl, min=-10.0, max=10.0)
    return kl


def compute_gspo_kl(log_probs, old_log_probs, mask, seq_ids, num_seqs):
    """GSPO: the sequence mean of (logp_old − logp), expanded to every token of the sequence."""
    return segment_mean_expand(old_log_probs.float() - log_probs.float(), mask, seq_ids, num_seqs)


def compute_opsm_mask(log_probs, old_log_probs, advantages, mask, seq_ids, num_seqs, delta: float):
    """Off-policy sequence masking: a token is dropped when ITS advantage is negative and the mean KL(old‖new) of its
    sequence exceeds delta (per-token test on the advantage, per-sequence test on the KL; with GRPO's constant advantage
    that drops whole sequences, with GAE advantages only the negative tokens — reference: loss/hub/math_utils.py:183-222).

    Returns (keep mask [R] float, Σ over sequences of the dropped-token fraction ÷ number of sequences)."""
    n_tok = segment_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
    seq_kl = segment_sum((old_log_probs.float() - log_probs.float()) * mask, seq_ids, num_seqs) / n_tok
    drop = ((advantages.float() < 0) & (seq_kl > delta)[seq_ids]).float()
    frac = (segment_sum(drop, seq_ids, num_seqs) / n_tok).sum() / max(num_seqs, 1)
    return 1.0 - drop, frac


def compute_policy_loss(ppo_kl, advantages, eps_clip: float, eps_clip_high: float, eps_clip_c: float | None = None):
    """PPO clipped surrogate on ppo_kl = logp_old − logp. Returns (per-token loss, clipfrac indicator)."""
    ratio = torch.exp(torch.clamp(-ppo_kl, min=-20.0, max=20.0))
    a = advantages.float()
    l1 = -ratio * a
    l2 = -torch.clamp(ratio, 1.0 - eps_clip, 1.0 + eps_clip_high) * a
    loss = torch.maximum(l1, l2)
    clipfrac = (l2 > l1).float()
    if eps_clip_c is not None:
        assert eps_clip_c > 1.0, "dual-clip constant must be > 1"
        l3 = -eps_clip_c * a
        loss = torch.where(a < 0, torch.minimum(l3, loss), loss)
    return loss, clipfrac


def compute_entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    return lse - (torch.softmax(lf, dim=-1) * lf).sum(-1)


# ---- returns / GAE -----------------------------------------------------------------------------

def _reverse_discounted_cumsum_padded(x: torch.Tensor, discount: float, chunk: int = 128) -> torch.Tensor:
    """y[:, t] = Σ_{j≥t} discount^(j−t) x[:, j] for x [B, L], scanned right-to-left in chunks.

    Inside a chunk the sum is one matmul with M[i, j] = discount^(j−i) (j ≥ i); across chunks a
    single carried column is folded in — the chunked scan of the reference's `chunked_gae`.
    """
    B, L = x.shape
    if L == 0:
        return x.clone()
    pad = (-L) % chunk
    xp = torch.nn.functional.pad(x.float(), (0, pad))
    n = xp.shape[1] // chunk
    ar = torch.arange(chunk, device=x.device)
    expo = (ar[None, :] - ar[:, None]).float()
    M = torch.where(expo >= 0, torch.pow(torch.tensor(discount, device=x.device, dtype=torch.float32), expo.clamp_min(0)),
                    torch.zeros((), device=x.device))          # [chunk(i), chunk(j)]
    carry_w = torch.pow(torch.tensor(discount, device=x.device, dtype=torch.float32), (chunk - ar).float())  # discount^(chunk−i)
    out = torch.empty_like(xp)
    carry = torch.zeros(B, device=x.device, dtype=torch.float32)
    for c in range(n - 1, -1, -1):
        seg = xp[:, c * chunk:(c + 1) * chunk]
        y = seg @ M.T + carry[:, None] * carry_w[None, :]
        out[:, c * chunk:(c + 1) * chunk] = y
        carry = y[:, 0]
    return out[:, :L]


def chunked_gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lambd: float, chunk: int = 128):
    """Batched GAE over right-padded [B, L] tensors. Returns (advantages, returns)."""
    nxt = torch.cat([values[:, 1:], torch.zeros_like(values[:, :1])], dim=1)
    delta = rewards.float() + gamma * nxt.float() - values.float()
    adv = _reverse_discounted_cumsum_padded(delta, gamma * lambd, chunk)
    return adv, adv + values.float()


def vanilla_gae(rewards, values, gamma, lambd):
    """Reference O(L) python scan, used as the oracle in tests."""
    B, L = rewards.shape
    adv = torch.zeros(B, L, dtype=torch.float32, device=rewards.device)
    last = torch.zeros(B, dtype=torch.float32, device=rewards.device)
    for t in range(L - 1, -1, -1):
        nv = values[:, t + 1].float() if t + 1 < L else torch.zeros(B, device=rewards.device)
        d = rewards[:, t].float() + gamma * nv - values[:, t].float()
        last = d + gamma * lambd * last
        adv[:, t] = last
    return adv, adv + values.float()


def pad_by_lengths(flat: torch.Tensor, lengths: list[int], pad_value: float = 0.0) -> torch.Tensor:
    B, L = len(lengths), (max(lengths) if lengths else 0)
    out = torch.full((B, L), pad_value, dtype=flat.dtype, device=flat.device)
    lens = torch.as_tensor(lengths, device=flat.device)
    m = torch.arange(L, device=flat.device)[None, :] < lens[:, None]
    out[m] = flat
    return out


def unpad_by_lengths(padded: torch.Tensor, lengths: list[int]) -> torch.Tensor:
    lens = torch.as_tensor(lengths, device=padded.device)
    m = torch.arange(padded.shape[1], device=padded.device)[None, :] < lens[:, None]
    return padded[m]


def masked_gae(token_rewards, values, loss_mask, lengths, gamma, lambd):
    """GAE over flat [R] tensors where masked-out tokens (tool output etc.) are skipped: the scan runs
    on the compressed sequence of unmasked tokens and results are scattered back (zeros elsewhere)."""
    keep = loss_mask > 0
    seq_ids = lengths_to_seq_ids(lengths, token_rewards.device)
    kept_lengths = segment_sum(keep.float(), seq_ids, len(lengths)).long().tolist()
    r = pad_by_lengths(token_rewards[keep].float(), kept_lengths)
    v = pad_by_lengths(values[keep].float(), kept_lengths)
    adv_p, ret_p = chunked_gae(r, v, gamma, lambd)
    adv = torch.zeros_like(token_rewards, dtype=torch.float32)
    ret = torch.zeros_like(token_rewards, dtype=torch.float32)
    adv[keep] = unpad_by_lengths(adv_p, kept_lengths)
    ret[keep] = unpad_by_lengths(ret_p, kept_lengths)
    return adv, ret


def discounted_returns(token_rewards, lengths, gamma):
    """REINFORCE++: per-token discounted return within each sequence (flat in, flat out)."""
    p = pad_by_lengths(token_rewards.float(), lengths)
    return unpad_by_lengths(_reverse_discounted_cumsum_padded(p, gamma), lengths)


# ---- whitening ---------------------------------------------------------------------------------

def masked_whiten(x: torch.Tensor, mask: torch.Tensor, group=None, shift_mean: bool = True, eps: float = 1e-8):
    """(x − mean)/std over unmasked tokens, statistics all-reduced over `group` (one [3] message:
    Σx, Σx², n — reference: miles/utils/distributed_utils.py:105-165)."""
    import torch.distributed as dist

    xf, m = x.float(), mask.float()
    stats = torch.stack([(xf * m).sum(), (xf * xf * m).sum(), m.sum()])
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(stats, group=group)
    n = stats[2].clamp_min(1.0)
    mean = stats[0] / n
    var = (stats[1] / n - mean * mean).clamp_min(0.0)
    var = var * n / (n - 1).clamp_min(1.0)  # unbiased
    out = (xf - mean) * torch.rsqrt(var + eps)
    if not shift_mean:
        out = out + mean
    return out
