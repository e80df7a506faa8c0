"""Stream the trainer's weights as buckets of HF-named full tensors.

For every parameter: pipeline owner broadcasts (PP) → tensor-parallel shards are all-gathered and
un-sharded (QKV by heads, gate/up halves) → experts are converted locally and gathered over the
expert-parallel group as one byte payload per bucket → names/layouts converted to HF → optional
quantisation (fp8 128×128 blocks or MXFP8 1×32) that adds `<name>_scale_inv` tensors.  Buckets are
cut at `--update-weight-buffer-size` bytes and never split an atomic group (q/k/v of one layer,
gate/up of one expert).  Reference: miles/backends/megatron_utils/update_weight/
hf_weight_iterator_direct.py:31-476 and expert_gather.py:29-164; every rank must drive the iterator
because it runs collectives.
"""
from __future__ import annotations

from typing import Iterator

import torch
import torch.distributed as dist

from ..models.convert import to_hf, unshard_tp
from .quantize import quantize_hf_tensors


def _all_gather_tp(t: torch.Tensor, ps) -> list[torch.Tensor]:
    if ps.tp_size == 1:
        return [t]
    parts = [torch.empty_like(t) for _ in range(ps.tp_size)]
    dist.all_gather(parts, t.contiguous(), group=ps.tp_group)
    return parts


def _gather_experts(t: torch.Tensor, ps) -> torch.Tensor:
    """[E_local, …] on each EP rank → [E, …] everywhere (byte payload all-gather)."""
    if ps.ep_size == 1:
        return t
    flat = t.contiguous().view(torch.uint8).reshape(-1)
    out = torch.empty(ps.ep_size * flat.numel(), dtype=torch.uint8, device=t.device)
    if t.is_cuda and dist.get_backend(ps.ep_group) == "nccl":
        dist.all_gather_into_tensor(out, flat, group=ps.ep_group)
    else:
        parts = [torch.empty_like(flat) for _ in range(ps.ep_size)]
        dist.all_gather(parts, flat, group=ps.ep_group)
        out = torch.cat(parts)
    return out.view(t.dtype).reshape(ps.ep_size * t.shape[0], *t.shape[1:])


def _pp_broadcast(name: str, t: torch.Tensor | None, shape, dtype, owner_pp: int, ps, device) -> torch.Tensor:
    if ps.pp_size == 1:
        return t
    buf = t.contiguous() if ps.pp_rank == owner_pp else torch.empty(shape, dtype=dtype, device=device)
    dist.broadcast(buf, src=ps.pp_ranks[owner_pp], group=ps.pp_group)
    return buf


def iter_full_tensors(actor) -> Iterator[tuple[str, torch.Tensor]]:
    """(our name, full tensor) for every parameter of the whole model, on every rank."""
    ps, cfg = actor.ps, actor.cfg
    local = dict(actor.named_weights())
    if ps.pp_size > 1:
        # exchange the (name, shape, dtype) manifests so non-owners can allocate receive buffers
        manifest = [(n, tuple(t.shape), t.dtype) for n, t in local.items()]
        all_m: list = [None] * ps.pp_size
        dist.all_gather_object(all_m, manifest, group=ps.pp_group)
        plan = [(n, s, d, stage) for stage, m in enumerate(all_m) for (n, s, d) in m]
    else:
        plan = [(n, tuple(t.shape), t.dtype, 0) for n, t in local.items()]
    for name, shape, dtype, stage in plan:
        t = _pp_broadcast(name, local.get(name), shape, dtype, stage, ps, actor.device)
        if t.dim() == 3 and name.endswith(("mlp.w13", "mlp.w2")):
            yield name, _gather_experts(t, ps)
        else:
            yield name, unshard_tp(name, _all_gather_tp(t, ps), cfg)


def quant_options_from_args(args, quant: str | None, cfg) -> dict:
    """Options of the packed export formats taken from the command line."""
    if quant == "nvfp4":
        return {"ignore": list(getattr(args, "export_quant_ignore", None) or []) + list(getattr(args, "extra_high_precision_layers_hf", None) or []),
                "four_over_six": bool(getattr(args, "nvfp4_four_over_six", False)), "num_layers": cfg.num_layers,
                "bf16_head": int(getattr(args, "num_layers_at_start_in_bf16", 0) or 0),
                "bf16_tail": int(getattr(args, "num_layers_at_end_in_bf16", 0) or 0),
                "all_linears": bool(getattr(args, "export_quant_all_linears", False))}
    if quant == "int4":
        return {"ignore": list(getattr(args, "export_quant_ignore", None) or []), "group_size": int(getattr(args, "int4_group_size", 32) or 32),
                "symmetric": not getattr(args, "int4_asymmetric", False)}
    return {}


def iter_hf_weights(actor, bucket_bytes: int | None = 512 << 20, quant: str | None = None
                    ) -> Iterator[list[tuple[str, torch.Tensor]]]:
    """Buckets of (hf_name, tensor). `quant` ∈ {None, 'fp8', 'mxfp8', 'nvfp4', 'int4'}."""
    qopts = quant_options_from_args(getattr(actor, "args", None), quant, actor.cfg)
    cfg = actor.cfg
    bucket: list[tuple[str, torch.Tensor]] = []
    size = 0
    for name, full in iter_full_tensors(actor):
        group = to_hf(name, full, cfg)
        if quant:
            group = quantize_hf_tensors(group, quant, **qopts)
        nb = sum(t.numel() * t.element_size() for _, t in group)
        if bucket_bytes is not None and bucket and size + nb > bucket_bytes:
            yield bucket
            bucket, size = [], 0
        # a stacked expert tensor may exceed the budget on its own: cut between experts (atomic = one expert)
        if bucket_bytes is not None and nb > bucket_bytes and len(group) > 3:
            for n, t in group:
                b = t.numel() * t.element_size()
                if bucket and size + b > bucket_bytes and not _splits_atomic(bucket[-1][0], n):
                    yield bucket
                    bucket, size = [], 0
                bucket.append((n, t))
                size += b
            continue
        bucket.extend(group)
        size += nb
    if bucket:
        yield bucket


def _splits_atomic(prev: str, nxt: str) -> bool:
    """True when cutting between prev and nxt would separate members of one atomic group."""
    def stem(n):
        for suf in ("gate_proj.weight", "up_proj.weight", "q_proj.weight", "k_proj.weight", "v_proj.weight",
                    "gate_proj.weight_scale_inv", "up_proj.weight_scale_inv"):
            if n.endswith(suf):
                return n[: -len(suf)]
        return None
    a, b = stem(prev), stem(nxt)
    return a is not None and a == b


def hf_named_weights_local(actor) -> dict[str, torch.Tensor]:
    """Convenience for single-rank tests: the full HF state dict."""
    out = {}
    for bucket in iter_hf_weights(actor, bucket_bytes=None):
        out.update(dict(bucket))
    return out
