"""Rollout samples → per-DP-rank train data → packed micro-batches.

* `convert_samples_to_train_data`: `Sample` list → dict of ragged lists with group-normalised
  rewards (reference: miles/ray/rollout/train_data_conversion.py:57-196).
* `split_train_data_by_dp`: round-robin or sequence-length-balanced (Karmarkar–Karp) partition
  (reference :342-473, miles/utils/seqlen_balancing.py).
* `make_micro_batches`: fixed `micro_batch_size` or dynamic token budget, micro-batch count
  equalised across DP ranks with one all-reduce(MAX) (reference: data/rollout.py:455-568).
* `pack_micro_batch`: THD packing — concatenated tokens padded to a multiple of `tp×128`,
  `cu_seqlens`, positions, response-aligned gather indices and loss masks
  (reference: data/rollout.py:168-381).
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ..types import Sample, Status
from ..utils.misc import load_function
from .advantages import normalize_group_rewards

PAD_MULTIPLE = 128

# bytes this module moved between host and device (what a step's end-to-end accounting reads)
TRANSFER = {"h2d_bytes": 0}


def to_device(values, dtype, device) -> torch.Tensor:
    """Host list / array → device tensor.  On CUDA the staging tensor is pinned (the caching host allocator reuses the
    pages) and the copy is asynchronous on the current stream."""
    t = values if isinstance(values, torch.Tensor) else torch.tensor(values, dtype=dtype)
    if torch.device(device).type != "cuda":
        return t.to(device)
    TRANSFER["h2d_bytes"] += t.numel() * t.element_size()
    return t.pin_memory().to(device, non_blocking=True)


# ---- samples → train data ----------------------------------------------------------------------

def convert_samples_to_train_data(args, samples: list[Sample] | list[list[Sample]]) -> dict[str, Any]:
    custom = getattr(args, "custom_convert_samples_to_train_data_path", None)
    if custom:
        return load_function(custom)(args, samples)
    if samples and isinstance(samples[0], list):
        group_sizes = [len(g) for g in samples]
        flat = [s for g in samples for s in g]
    else:
        flat = list(samples)
        n = getattr(args, "n_samples_per_prompt", 1)
        group_sizes = [n] * (len(flat) // n) + ([len(flat) % n] if len(flat) % n else [])
    # samples marked remove_sample stay in the batch (their reward still counts in the group statistics and the batch and
    # shard sizes stay fixed); only their loss mask is zeroed below
    raw = torch.tensor([s.get_reward_value(getattr(args, "reward_key", None)) for s in flat], dtype=torch.float32)
    post = getattr(args, "custom_reward_post_process_path", None)
    if post:
        rewards = torch.as_tensor(load_function(post)(args, flat), dtype=torch.float32)
    else:
        rewards = normalize_rewards_by_rollout(args, flat, raw, group_sizes)
    data: dict[str, Any] = {
        "tokens": [list(s.tokens) for s in flat],
        "response_lengths": [s.response_length for s in flat],
        "total_lengths": [len(s.tokens) for s in flat],
        "rewards": rewards.tolist(),
        "raw_reward": raw.tolist(),
        "truncated": [1 if s.status == Status.TRUNCATED else 0 for s in flat],
        "loss_masks": [[0] * s.response_length if s.remove_sample else
                       (list(s.loss_mask) if s.loss_mask is not None else [1] * s.response_length) for s in flat],
        "sample_indices": [s.index for s in flat],
        "rollout_ids": [s.rollout_id if s.rollout_id is not None else s.index for s in flat],
        "prompt_group_sizes": group_sizes,
    }
    for s, lm in zip(flat, data["loss_masks"]):
        assert s.loss_mask is None or len(s.loss_mask) == s.response_length, \
            f"loss_mask length {len(s.loss_mask)} != response_length {s.response_length}"
        assert len(lm) == s.response_length, f"loss_mask length {len(lm)} != response_length {s.response_length}"
    if all(s.rollout_log_probs is not None for s in flat) and flat:
        data["rollout_log_probs"] = [list(s.rollout_log_probs) for s in flat]
    if all(s.rollout_routed_experts is not None for s in flat) and flat:
        data["rollout_routed_experts"] = [np.asarray(s.rollout_routed_experts, dtype=np.int32) for s in flat]
    if all(s.teacher_log_probs is not None for s in flat) and flat:
        data["teacher_log_probs"] = [list(s.teacher_log_probs) for s in flat]
    if all(s.opd_reverse_kl is not None for s in flat) and flat:
        data["opd_reverse_kl"] = [list(s.opd_reverse_kl) for s in flat]
    if any(s.weight_versions for s in flat):
        data["weight_versions"] = [s.oldest_weight_version for s in flat]
    if any(getattr(s, "multimodal_train_inputs", None) for s in flat):
        data["multimodal_train_inputs"] = [s.multimodal_train_inputs for s in flat]
    # per-rollout mask sums: siblings of one rollout (same rollout_id) share a denominator
    sums: dict[Any, int] = {}
    for rid, lm in zip(data["rollout_ids"], data["loss_masks"]):
        sums[rid] = sums.get(rid, 0) + int(sum(lm))
    data["rollout_mask_sums"] = [sums[rid] for rid in data["rollout_ids"]]
    return data


def normalize_rewards_by_rollout(args, flat: list[Sample], raw: torch.Tensor, group_sizes: list[int]) -> torch.Tensor:
    """Group normalisation with one vote per rollout: segments of one rollout (same `rollout_id`, e.g. the turns of a
    multi-turn trajectory split into several training rows) carry one shared reward, which enters the prompt group's
    mean / std once and is broadcast back to every segment; siblings with different rewards are an error
    (reference: miles/ray/rollout/train_data_conversion.py:275-322)."""
    est = args.advantage_estimator
    if est not in ("grpo", "gspo", "reinforce_plus_plus_baseline") or not getattr(args, "rewards_normalization", True):
        return raw.float()
    out = torch.empty(len(flat), dtype=torch.float32)
    off = 0
    for n in group_sizes:
        keys: dict[Any, list[int]] = {}
        for i in range(off, off + n):
            s = flat[i]
            key = s.rollout_id if s.rollout_id is not None else (s.index if s.index is not None else ("row", i))
            keys.setdefault(key, []).append(i)
        shared = []
        for key, rows in keys.items():
            vals = [float(raw[i]) for i in rows]
            if any(v != vals[0] for v in vals[1:]):
                raise ValueError(f"all samples of rollout {key!r} must share one reward; rows {rows} have rewards {vals}")
            shared.append(vals[0])
        normed = normalize_group_rewards(args, torch.tensor(shared, dtype=torch.float32), [len(shared)])
        for (key, rows), v in zip(keys.items(), normed.tolist()):
            for i in rows:
                out[i] = v
        off += n
    return out


_PER_SAMPLE_KEYS = ("tokens", "response_lengths", "total_lengths", "rewards", "raw_reward", "truncated", "loss_masks",
                    "sample_indices", "rollout_ids", "rollout_log_probs", "rollout_routed_experts",
                    "teacher_log_probs", "opd_reverse_kl", "weight_versions", "rollout_mask_sums", "advantages",
                    "multimodal_train_inputs", "witness_ids")


def karmarkar_karp(lengths: list[int], k: int, equal_size: bool = True) -> list[list[int]]:
    """Largest-differencing partition of indices into k sets with near-equal total length."""
    n = len(lengths)
    if k == 1:
        return [list(range(n))]
    order = sorted(range(n), key=lambda i: -lengths[i])
    if equal_size:
        # process in rounds of k items; within a round, longest goes to the currently lightest set
        parts: list[list[int]] = [[] for _ in range(k)]
        sums = [0] * k
        for r in range(0, n, k):
            chunk = order[r:r + k]
            light = sorted(range(k), key=lambda j: sums[j])
            for j, i in zip(light, chunk):
                parts[j].append(i)
                sums[j] += lengths[i]
        return parts
    heap = [(0, j) for j in range(k)]
    heapq.heapify(heap)
    parts = [[] for _ in range(k)]
    for i in order:
        s, j = heapq.heappop(heap)
        parts[j].append(i)
        heapq.heappush(heap, (s + lengths[i], j))
    return parts


def split_train_data_by_dp(args, data: dict[str, Any], dp_size: int) -> list[dict[str, Any]]:
    n = len(data["tokens"])
    if getattr(args, "balance_data", False):
        parts = karmarkar_karp(data["total_lengths"], dp_size, equal_size=True)
        parts = [sorted(p) for p in parts]
    else:
        parts = [list(range(r, n, dp_size)) for r in range(dp_size)]
    out = []
    for p in parts:
        shard = {"partition": p}
        for k, v in data.items():
            if k in _PER_SAMPLE_KEYS:
                shard[k] = [v[i] for i in p]
            else:
                shard[k] = v
        out.append(shard)
    return out


# ---- micro-batching ----------------------------------------------------------------------------

def make_micro_batches(args, total_lengths: list[int], *, dp_group=None, cp_size: int = 1,
                       max_tokens: int | None = None, vpp_multiple: int = 1) -> list[list[int]]:
    """Partition local sample indices into micro-batches; every DP rank ends with the same count."""
    n = len(total_lengths)
    if getattr(args, "use_dynamic_batch_size", False):
        budget = (max_tokens or args.max_tokens_per_gpu) * cp_size
        # first-fit decreasing for the count, then balanced partition at that count
        bins: list[int] = []
        for L in sorted(total_lengths, reverse=True):
            for j in range(len(bins)):
                if bins[j] + L <= budget:
                    bins[j] += L
                    break
            else:
                bins.append(L)
        num = max(1, len(bins))
    else:
        mbs = getattr(args, "micro_batch_size", 1)
        num = max(1, (n + mbs - 1) // mbs)
    if dp_group is not None and dist.is_initialized() and dist.get_world_size(dp_group) > 1:
        dev = "cuda" if dist.get_backend(dp_group) == "nccl" else "cpu"
        t = torch.tensor([num], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        num = int(t.item())
    if vpp_multiple > 1:
        num = (num + vpp_multiple - 1) // vpp_multiple * vpp_multiple
    # every DP rank returns exactly `num` parts (never fewer than the reduced count: layers with collectives inside the
    # forward must run the same number of times everywhere); a rank with too few samples pads with empty parts
    if n == 0:
        return [[] for _ in range(num)]
    if getattr(args, "use_dynamic_batch_size", False):
        parts = karmarkar_karp(total_lengths, num, equal_size=False)
        parts = [sorted(p) for p in parts]
    else:
        mbs = (n + num - 1) // num
        parts = [list(range(i, min(n, i + mbs))) for i in range(0, n, mbs)]
    while len(parts) < num:
        parts.append([])
    return parts


# ---- packing -----------------------------------------------------------------------------------

@dataclass
class PackedBatch:
    tokens: torch.Tensor            # int32 [T_pad]
    positions: torch.Tensor         # int32 [T_pad]
    cu_seqlens: torch.Tensor        # int32 [B+1(+1 for the padding pseudo-sequence)]
    max_seqlen: int
    total_lengths: list[int]
    response_lengths: list[int]
    gather_index: torch.Tensor      # int64 [R]: hidden-state row predicting each response token
    targets: torch.Tensor           # int64 [R]: the response token ids
    loss_mask: torch.Tensor         # float [R]
    seq_ids: torch.Tensor           # int64 [R]
    sample_index: list[int] = field(default_factory=list)   # indices into the rank-local shard
    replay_topk: torch.Tensor | None = None  # int32 [T_pad, L_moe, k]
    num_real_tokens: int = 0
    mm_inputs: dict | None = None   # vision-language: {"patches": [N, patch_dim], "grid_thw": [n_images, 3]} of the packed samples


def pack_micro_batch(shard: dict[str, Any], idx: list[int], device, *, pad_multiple: int = PAD_MULTIPLE,
                     with_replay: bool = False) -> PackedBatch:
    toks, pos, cu = [], [], [0]
    gather, targets, mask, seq_ids = [], [], [], []
    total_lengths, response_lengths = [], []
    off = 0
    for j, i in enumerate(idx):
        t = shard["tokens"][i]
        L, R = len(t), shard["response_lengths"][i]
        P = L - R
        toks.extend(t)
        pos.extend(range(L))
        # the logit at position p predicts token p+1: response tokens P..L-1 ← rows P-1..L-2
        gather.extend(range(off + P - 1, off + L - 1))
        targets.extend(t[P:])
        mask.extend(shard["loss_masks"][i])
        seq_ids.extend([j] * R)
        off += L
        cu.append(off)
        total_lengths.append(L)
        response_lengths.append(R)
    real = off
    pad = (-off) % pad_multiple if pad_multiple > 1 else 0
    if off == 0:
        pad = pad_multiple
    if pad:
        toks.extend([0] * pad)
        pos.extend(range(pad))
        off += pad
        cu.append(off)  # padding forms its own sequence so it never attends to real tokens
    max_len = max([b - a for a, b in zip(cu[:-1], cu[1:])], default=0)
    replay = None
    if with_replay and "rollout_routed_experts" in shard:
        rows = []
        for i in idx:
            re = torch.from_numpy(np.asarray(shard["rollout_routed_experts"][i], dtype=np.int32))
            L = len(shard["tokens"][i])
            # engine records routing for tokens 0..L-2 (the last token is never fed back); pad one row
            fill = torch.full((L - re.shape[0],) + tuple(re.shape[1:]), -1, dtype=torch.int32)
            rows.append(torch.cat([re, fill], 0))
        if rows:
            body = torch.cat(rows, 0)
            if pad:
                body = torch.cat([body, torch.full((pad,) + tuple(body.shape[1:]), -1, dtype=torch.int32)], 0)
            replay = to_device(body, torch.int32, device)
    mm = None
    if shard.get("multimodal_train_inputs") is not None:
        # per-sample {"patches", "grid_thw"} in sample order = the order of the image placeholder tokens in the packed stream
        parts = [shard["multimodal_train_inputs"][i] for i in idx]
        parts = [p for p in parts if p and p.get("patches") is not None and len(p["patches"])]
        if parts:
            mm = {"patches": torch.cat([torch.as_tensor(p["patches"]) for p in parts], 0).to(device),
                  "grid_thw": torch.cat([torch.as_tensor(p["grid_thw"]).view(-1, 3) for p in parts], 0).to(device)}
    return PackedBatch(
        mm_inputs=mm,
        tokens=to_device(toks, torch.int32, device),
        positions=to_device(pos, torch.int32, device),
        cu_seqlens=to_device(cu, torch.int32, device),
        max_seqlen=max_len,
        total_lengths=total_lengths,
        response_lengths=response_lengths,
        gather_index=to_device(gather, torch.int64, device),
        targets=to_device(targets, torch.int64, device),
        loss_mask=to_device(mask, torch.float32, device),
        seq_ids=to_device(seq_ids, torch.int64, device),
        sample_index=list(idx),
        replay_topk=replay,
        num_real_tokens=real,
    )


def flat_per_token(shard: dict[str, Any], key: str, idx: list[int], device, dtype=torch.float32) -> torch.Tensor | None:
    if key not in shard:
        return None
    vals: list = []
    for i in idx:
        vals.extend(shard[key][i])
    return to_device(vals, dtype, device)
