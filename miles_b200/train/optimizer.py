"""Distributed (ZeRO-1 style) Adam over flat parameter/gradient buffers.

Layout.  Parameters of one *reduction domain* (dense params → the data-parallel group; expert
params → the expert-data-parallel group) are re-pointed into one contiguous buffer in the compute
dtype; gradients accumulate in an fp32 `main_grad` buffer of the same layout through
post-accumulate hooks; fp32 master weights and both Adam moments exist only for this rank's
contiguous shard of the buffer.  One step is

    reduce-scatter(main_grad, SUM) → clip → Adam on the shard → all-gather(param buffer)

which is what the reference gets from Megatron's DDP + distributed optimizer
(miles/backends/megatron_utils/model.py:565-671, :686-701).  On CUDA with a fabric the three stages
are ONE kernel (`fused_rs_adam_ag`): each rank sums its shard of every peer's gradient buffer
through NVLink loads, applies Adam, and stores the new bf16 parameters into every peer's parameter
buffer.  On CPU (gloo) and in the baseline mode the stages are separate collectives.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Iterable

import torch
import torch.distributed as dist

from .. import ops

ALIGN = 256  # elements; keeps every shard 16-byte aligned for vector/TMA access in any dtype


@dataclass
class _Domain:
    name: str
    params: list[torch.nn.Parameter]
    group: Any
    group_size: int
    group_rank: int
    param_buf: torch.Tensor = None      # compute dtype, [N_pad]
    grad_buf: torch.Tensor = None       # fp32, [N_pad]
    master: torch.Tensor = None         # fp32 shard
    exp_avg: torch.Tensor = None
    exp_avg_sq: torch.Tensor = None
    shard: tuple[int, int] = (0, 0)
    numel: int = 0
    decay_mask: torch.Tensor | None = None  # fp32 shard, 1 where weight decay applies
    nvme: Any = None                    # NvmeStreamAdam holding this shard's state in files (then master / moments are file-backed views)
    names: list[str] = None             # parameter names, in buffer order
    offsets: list[int] = None           # element offset of each parameter in the flat buffers


class DistributedAdam:
    def __init__(self, named_params: Iterable[tuple[str, torch.nn.Parameter]], *, lr: float, betas=(0.9, 0.98),
                 eps: float = 1e-8, weight_decay: float = 0.0, clip_grad: float = 1.0, ps=None,
                 allocator=None, moments_dtype=torch.float32, state_allocator=None, nvme_dir: str | None = None,
                 nvme_bucket_numel: int = 64 << 20):
        self.lr, self.betas, self.eps, self.weight_decay, self.clip_grad = lr, betas, eps, weight_decay, clip_grad
        self.ps = ps
        self.step_count = 0
        self.allocator = allocator
        # where the fp32 master weights and the Adam moments live: None → ordinary tensors; a callable (n, dtype, device, tag)
        # → e.g. the VMM arena, whose physical pages can be released for the rollout phase at stable addresses
        self.state_allocator = state_allocator
        # fp32 master weights and Adam moments of this rank's shards in FILES under this directory, streamed through the
        # device bucket by bucket at every step (train/nvme_stream.py): for state that fits neither HBM nor host memory
        self.nvme_dir, self.nvme_bucket_numel = nvme_dir, nvme_bucket_numel
        named = [(n, p) for n, p in named_params if p.requires_grad]
        dense = [(n, p) for n, p in named if not _is_expert(n)]
        expert = [(n, p) for n, p in named if _is_expert(n)]
        self.domains: list[_Domain] = []
        if dense:
            g, gs, gr = (ps.dp_cp_group, ps.dp_cp_size, ps.dp_rank * ps.cp_size + ps.cp_rank) if ps else (None, 1, 0)
            self.domains.append(self._build("dense", dense, g, gs, gr, moments_dtype))
        if expert:
            g, gs, gr = (ps.edp_group, ps.edp_size, ps.edp_rank) if ps else (None, 1, 0)
            self.domains.append(self._build("expert", expert, g, gs, gr, moments_dtype))
        self._hooks = []
        for d in self.domains:
            for p in d.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(_accumulate_hook))

    # ---- construction --------------------------------------------------------------------
    def _alloc(self, n, dtype, device, tag):
        if self.allocator is not None:
            return self.allocator(n, dtype, device, tag)
        return torch.zeros(n, dtype=dtype, device=device)

    def _build(self, name, named, group, gsize, grank, moments_dtype) -> _Domain:
        params = [p for _, p in named]
        device, dtype = params[0].device, params[0].dtype
        offs, total = [], 0
        for p in params:
            offs.append(total)
            total += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        unit = ALIGN * gsize
        n_pad = (total + unit - 1) // unit * unit
        d = _Domain(name, params, group, gsize, grank, numel=n_pad, names=[n for n, _ in named], offsets=offs)
        d.param_buf = self._alloc(n_pad, dtype, device, f"{name}.param")
        d.grad_buf = self._alloc(n_pad, torch.float32, device, f"{name}.grad")
        decay = torch.zeros(n_pad, dtype=torch.float32, device=device)
        for (pname, p), o in zip(named, offs):
            view = d.param_buf[o:o + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.main_grad = d.grad_buf[o:o + p.numel()].view_as(p)
            if p.dim() >= 2:
                decay[o:o + p.numel()] = 1.0
        s = n_pad // gsize
        d.shard = (grank * s, (grank + 1) * s)
        d.decay_mask = decay[d.shard[0]:d.shard[1]].clone()
        if self.nvme_dir is not None:
            from .nvme_stream import NvmeStreamAdam

            rank = dist.get_rank() if dist.is_initialized() else 0
            d.nvme = NvmeStreamAdam(d.param_buf[d.shard[0]:d.shard[1]], os.path.join(self.nvme_dir, name), lr=self.lr, betas=self.betas,
                                    eps=self.eps, weight_decay=self.weight_decay, bucket_numel=self.nvme_bucket_numel, rank=rank,
                                    decay_mask=d.decay_mask)
            # file-backed views: everything that reads or writes the optimizer state (checkpoints, resets) goes to the files
            d.master, d.exp_avg, d.exp_avg_sq = d.nvme.tensor("master"), d.nvme.tensor("exp_avg"), d.nvme.tensor("exp_avg_sq")
        elif self.state_allocator is not None:
            d.master = self.state_allocator(s, torch.float32, device, f"{name}.master")
            d.master.copy_(d.param_buf[d.shard[0]:d.shard[1]])
            d.exp_avg = self.state_allocator(s, moments_dtype, device, f"{name}.exp_avg").zero_()
            d.exp_avg_sq = self.state_allocator(s, moments_dtype, device, f"{name}.exp_avg_sq").zero_()
        else:
            d.master = d.param_buf[d.shard[0]:d.shard[1]].float().clone()
            d.exp_avg = torch.zeros(s, dtype=moments_dtype, device=device)
            d.exp_avg_sq = torch.zeros(s, dtype=moments_dtype, device=device)
        if group is not None:
            from ..parallel.reloadable import REGISTRY

            REGISTRY.bind(d, "group")                  # the handle follows a release / reload of the process groups
        return d

    # ---- step ----------------------------------------------------------------------------
    def zero_grad(self):
        for d in self.domains:
            d.grad_buf.zero_()
            for p in d.params:
                p.grad = None

    def _reduce_scatter(self, d: _Domain) -> torch.Tensor:
        lo, hi = d.shard
        if d.group_size == 1:
            return d.grad_buf[lo:hi]
        if d.grad_buf.is_cuda and dist.get_backend(d.group) == "nccl":
            out = d.grad_buf[lo:hi]
            dist.reduce_scatter_tensor(out, d.grad_buf, op=dist.ReduceOp.SUM, group=d.group)
            return out
        dist.all_reduce(d.grad_buf, op=dist.ReduceOp.SUM, group=d.group)  # gloo has no reduce_scatter
        return d.grad_buf[lo:hi]

    def _all_gather(self, d: _Domain):
        if d.group_size == 1:
            return
        lo, hi = d.shard
        if d.param_buf.is_cuda and dist.get_backend(d.group) == "nccl":
            dist.all_gather_into_tensor(d.param_buf, d.param_buf[lo:hi].clone(), group=d.group)
        else:
            parts = [torch.empty(hi - lo, dtype=d.param_buf.dtype, device=d.param_buf.device) for _ in range(d.group_size)]
            dist.all_gather(parts, d.param_buf[lo:hi].contiguous(), group=d.group)
            d.param_buf.copy_(torch.cat(parts))

    def grad_norm(self, shards: list[torch.Tensor]) -> torch.Tensor:
        """Global L2 norm: Σ over shards, all-reduced over every rank that holds distinct gradient."""
        sq = torch.zeros((), dtype=torch.float32, device=shards[0].device)
        for d, g in zip(self.domains, shards):
            sq = sq + self._owned_sq_norm(d, g)
        if self.ps is not None and self.ps.world_size > 1 and dist.is_initialized():
            dist.all_reduce(sq, op=dist.ReduceOp.SUM)
        return sq.sqrt()

    def _owned_sq_norm(self, d: _Domain, g: torch.Tensor) -> torch.Tensor:
        # parameters replicated across tensor-parallel ranks (norm weights, router) must count once
        ps = self.ps
        w = 1.0
        if ps is not None and ps.tp_size > 1 and d.name == "dense":
            rep = getattr(self, "_tp_replicated_mask", {}).get(d.name)
            if rep is not None and ps.tp_rank != 0:
                return (g.float() * (1.0 - rep)).pow(2).sum()
        return g.float().pow(2).sum() * w

    def mark_tp_replicated(self, names_replicated: set[str], named_params):
        """Record which flat ranges are TP-replicated so the grad norm counts them once."""
        self._tp_replicated_mask = {}
        name_of = {id(p): n for n, p in named_params}
        for d in self.domains:
            m = torch.zeros(d.numel, dtype=torch.float32, device=d.param_buf.device)
            base = d.param_buf.data_ptr()
            for p in d.params:
                if name_of.get(id(p)) in names_replicated:
                    o = (p.data.data_ptr() - base) // d.param_buf.element_size()
                    m[o:o + p.numel()] = 1.0
            self._tp_replicated_mask[d.name] = m[d.shard[0]:d.shard[1]].clone()

    @torch.no_grad()
    def step(self, lr: float | None = None) -> dict:
        lr = self.lr if lr is None else lr
        self.step_count += 1
        fused = self._try_fused_step(lr)
        if fused is not None:
            return fused
        shards = [self._reduce_scatter(d) for d in self.domains]
        norm = self.grad_norm(shards)
        scale = 1.0
        if self.clip_grad and self.clip_grad > 0:
            scale = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0)
        b1, b2 = self.betas
        for d, g in zip(self.domains, shards):
            lo, hi = d.shard
            if d.nvme is not None:
                d.nvme.step_count = self.step_count - 1
                d.nvme.step(g, grad_scale=float(scale), lr=lr)
            else:
                _adam_shard(d, g, lr, b1, b2, self.eps, self.weight_decay, self.step_count, scale, d.param_buf[lo:hi])
            self._all_gather(d)
        return {"grad_norm": float(norm)}

    def _try_fused_step(self, lr):
        ps = self.ps
        if ps is None or ps.fabric is None or not ps.fused or self.nvme_dir is not None:
            return None
        from ..parallel import dp as dp_fused
        return dp_fused.fused_step(self, lr)

    # ---- state ---------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {
            "step": self.step_count,
            "domains": {d.name: {"master": d.master.cpu(), "exp_avg": d.exp_avg.cpu(), "exp_avg_sq": d.exp_avg_sq.cpu(),
                                 "shard": d.shard, "numel": d.numel} for d in self.domains},
        }

    def load_state_dict(self, sd: dict):
        self.step_count = sd["step"]
        for d in self.domains:
            s = sd["domains"][d.name]
            assert tuple(s["shard"]) == tuple(d.shard) and s["numel"] == d.numel, "optimizer shard layout changed"
            d.master.copy_(s["master"])
            d.exp_avg.copy_(s["exp_avg"])
            d.exp_avg_sq.copy_(s["exp_avg_sq"])

    def reload_master_from_params(self):
        """After loading model weights: refresh fp32 master from the (new) parameter buffer."""
        for d in self.domains:
            if d.nvme is not None:
                d.nvme.reload_master()
                continue
            d.master.copy_(d.param_buf[d.shard[0]:d.shard[1]].float())

    def reset_state(self):
        for d in self.domains:
            d.exp_avg.zero_()
            d.exp_avg_sq.zero_()
        self.step_count = 0

    def release_grads(self):
        """Free the fp32 gradient buffers (they are zero between steps); `restore_grads` re-creates them."""
        for d in self.domains:
            if d.grad_buf is None or getattr(d.grad_buf, "_symmetric", False):
                continue  # symmetric-heap buffers stay mapped for the peers
            self._grad_offsets = getattr(self, "_grad_offsets", {})
            base = d.grad_buf.data_ptr()
            self._grad_offsets[d.name] = [(p.main_grad.data_ptr() - base) // 4 for p in d.params]
            for p in d.params:
                p.main_grad = None
            d.grad_buf = None

    def restore_grads(self):
        for d in self.domains:
            if d.grad_buf is not None:
                continue
            d.grad_buf = torch.zeros(d.numel, dtype=torch.float32, device=d.param_buf.device)
            for p, o in zip(d.params, self._grad_offsets[d.name]):
                p.main_grad = d.grad_buf[o:o + p.numel()].view_as(p)

    def tensors_by_tag(self) -> dict[str, list[torch.Tensor]]:
        out = {"optimizer": [], "grad": [], "param": []}
        for d in self.domains:
            if d.nvme is None:                       # file-backed state occupies no device memory: nothing to move on sleep
                out["optimizer"] += [d.master, d.exp_avg, d.exp_avg_sq]
            out["grad"].append(d.grad_buf)
            out["param"].append(d.param_buf)
        return out


def _adam_shard(d: _Domain, g, lr, b1, b2, eps, wd, step, scale, param_out):
    """AdamW on one shard; weight decay only where `decay_mask` is 1 (matrices, not norms/biases)."""
    if g.is_cuda:
        ops._k().adamw_step_masked(d.master, g, d.exp_avg, d.exp_avg_sq, d.decay_mask, lr, b1, b2, eps, wd, step,
                                   scale, param_out)
        return
    gs = g.float() * scale
    m, v = d.exp_avg.float(), d.exp_avg_sq.float()
    m.mul_(b1).add_(gs, alpha=1 - b1)
    v.mul_(b2).addcmul_(gs, gs, value=1 - b2)
    d.exp_avg.copy_(m)
    d.exp_avg_sq.copy_(v)
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    d.master.mul_(1 - lr * wd * d.decay_mask).addcdiv_(m / bc1, denom, value=-lr)
    param_out.copy_(d.master)


def _accumulate_hook(p: torch.nn.Parameter):
    if p.grad is not None:
        p.main_grad.add_(p.grad)
        p.grad = None


def _is_expert(name: str, module_names: set[str] | None = None) -> bool:
    """Expert weights are the `w13`/`w2` of a layer whose MLP also owns a `router`."""
    return name in EXPERT_PARAM_NAMES


# filled by `mark_expert_params(model)` before the optimizer is built
EXPERT_PARAM_NAMES: set[str] = set()


def mark_expert_params(model: torch.nn.Module) -> set[str]:
    from ..models.qwen3 import MoEFFN

    EXPERT_PARAM_NAMES.clear()
    for mname, mod in model.named_modules():
        if isinstance(mod, MoEFFN):
            EXPERT_PARAM_NAMES.add(f"{mname}.w13")
            EXPERT_PARAM_NAMES.add(f"{mname}.w2")
    return set(EXPERT_PARAM_NAMES)


class LRScheduler:
    def __init__(self, base_lr, min_lr=0.0, warmup=0, decay_iters=None, style="constant"):
        self.base_lr, self.min_lr, self.warmup, self.decay_iters, self.style = base_lr, min_lr, warmup, decay_iters, style
        self.it = 0

    def get(self) -> float:
        it = self.it
        if self.warmup and it < self.warmup:
            return self.base_lr * (it + 1) / self.warmup
        if self.style == "constant" or not self.decay_iters:
            return self.base_lr
        t = min(1.0, (it - self.warmup) / max(1, self.decay_iters - self.warmup))
        if self.style == "linear":
            return self.min_lr + (self.base_lr - self.min_lr) * (1 - t)
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * t))

    def step(self):
        self.it += 1

    def state_dict(self):
        return {"it": self.it}

    def load_state_dict(self, sd):
        self.it = sd["it"]
