"""`--train-backend fsdp`: parameters sharded per decoder layer with PyTorch FSDP2 (`fully_shard`).

The reference's FSDP backend shards each `_no_split_modules` layer and then the root over a `dp_replicate × dp_shard`
mesh, keeps fp32 sharded parameters, computes in bf16 and reduces gradients in fp32
(miles/backends/fsdp_utils/actor.py:417-462, parallel.py:14-43).  The same here: every `DecoderLayer` and then the root
are wrapped, a layer's parameters are all-gathered right before its forward / backward and freed after it, gradients
are reduce-scattered, and AdamW runs on the shards.  `--fsdp-dp-replicate R` makes the mesh `R × (dp / R)` (HSDP:
shard inside a group, all-reduce across groups).

This is the memory-lean alternative to the default trainer (flat symmetric buffers, ZeRO-1 optimizer sharding with the
fused reduce-scatter + Adam + all-gather kernel); it is meant for dense models that do not fit replicated.  It runs with
tensor / expert / pipeline / context parallel sizes of 1, and the in-process engine keeps its own copy of the weights,
fed by the HF-named tensor stream (`named_weights` gathers full tensors).

`FsdpOptimizer` gives the trainer the interface it uses of `DistributedAdam`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _is_dtensor(t) -> bool:
    from torch.distributed.tensor import DTensor

    return isinstance(t, DTensor)


def local_data(p: torch.Tensor) -> torch.Tensor:
    """The locally stored part of a parameter (the shard of an FSDP parameter, the tensor itself otherwise)."""
    d = p.data if isinstance(p, torch.nn.Parameter) else p
    return d.to_local() if _is_dtensor(d) else d


def full_data(p: torch.Tensor) -> torch.Tensor:
    """The whole parameter on every rank (collective for FSDP parameters)."""
    d = p.data if isinstance(p, torch.nn.Parameter) else p
    return d.full_tensor() if _is_dtensor(d) else d


def copy_into(p: torch.nn.Parameter, full: torch.Tensor):
    """p ← full (the un-sharded value); an FSDP parameter takes its own slice."""
    if _is_dtensor(p.data):
        from torch.distributed.tensor import distribute_tensor

        src = distribute_tensor(full.to(device=p.device, dtype=p.dtype), p.data.device_mesh, p.data.placements)
        p.data.to_local().copy_(src.to_local())
    else:
        p.data.copy_(full)


def shard_model(model: torch.nn.Module, ps, device, dp_replicate: int = 1, compute_dtype=None):
    """Wrap every decoder layer and the root with `fully_shard` over the data-parallel ranks.  Returns the mesh."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    assert ps.tp_size == ps.pp_size == ps.cp_size == 1 and ps.ep_size == 1, "the FSDP backend shards over data parallelism only"
    world = dist.get_world_size() if dist.is_initialized() else 1
    kind = "cuda" if torch.device(device).type == "cuda" else "cpu"
    if dp_replicate > 1:
        assert world % dp_replicate == 0, "--fsdp-dp-replicate must divide the number of ranks"
        mesh = init_device_mesh(kind, (dp_replicate, world // dp_replicate), mesh_dim_names=("replicate", "shard"))
    else:
        mesh = init_device_mesh(kind, (world,), mesh_dim_names=("shard",))
    kw = {"mesh": mesh}
    if compute_dtype is not None and compute_dtype != next(model.parameters()).dtype:
        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=compute_dtype, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, **kw)
    fully_shard(model, **kw)
    return mesh


class FsdpOptimizer:
    """AdamW over the FSDP shards behind the part of `DistributedAdam`'s interface the trainer uses."""

    domains: list = []          # no flat gradient buffers (independent-DP exchange is not available with this backend)

    def __init__(self, named_params, *, lr, betas, eps, weight_decay, clip_grad):
        self.named = list(named_params)
        self.params = [p for _, p in self.named]
        self.lr, self.clip_grad = lr, clip_grad
        decay = [p for p in self.params if p.dim() >= 2]
        no_decay = [p for p in self.params if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
                                     lr=lr, betas=betas, eps=eps)
        self.step_count = 0

    def zero_grad(self):
        self.opt.zero_grad(set_to_none=True)

    def step(self, lr: float | None = None) -> dict:
        lr = self.lr if lr is None else lr
        for g in self.opt.param_groups:
            g["lr"] = lr
        with_grad = [p for p in self.params if p.grad is not None]
        max_norm = self.clip_grad if (self.clip_grad and self.clip_grad > 0) else float("inf")
        norm = torch.nn.utils.clip_grad_norm_(with_grad, max_norm)
        norm = norm.full_tensor() if _is_dtensor(norm) else norm
        self.opt.step()
        self.step_count += 1
        return {"grad_norm": float(norm)}

    # ---- checkpoint: each rank keeps its own shards -------------------------------------------------------------
    def state_dict(self) -> dict:
        state = {}
        for n, p in self.named:
            st = self.opt.state.get(p)
            if st:
                state[n] = {k: (local_data(v).clone() if torch.is_tensor(v) and v.dim() > 0 else v) for k, v in st.items()}
        return {"state": state, "step_count": self.step_count}

    def load_state_dict(self, sd: dict):
        if not self.opt.state:                       # create the moment tensors (a step with zero gradients and lr 0)
            for p in self.params:
                p.grad = torch.zeros_like(p)
            for g in self.opt.param_groups:
                g["lr"] = 0.0
            self.opt.step()
            self.zero_grad()
        for n, p in self.named:
            if n not in sd["state"]:
                continue
            st = self.opt.state[p]
            for k, v in sd["state"][n].items():
                if torch.is_tensor(v) and v.dim() > 0:
                    local_data(st[k]).copy_(v)
                elif torch.is_tensor(st.get(k)):
                    st[k].fill_(float(v))
                else:
                    st[k] = v
        self.step_count = sd.get("step_count", 0)

    # ---- no flat buffers to manage ----------------------------------------------------------------------------------
    def reload_master_from_params(self):
        pass

    def reset_state(self):
        self.opt.state.clear()

    def mark_tp_replicated(self, *a, **k):
        pass

    def release_grads(self):
        self.zero_grad()

    def restore_grads(self):
        pass

    def tensors_by_tag(self) -> dict:
        """The local moment shards (what `sleep` moves to host memory during the rollout phase)."""
        moments = [local_data(v) for st in self.opt.state.values() for v in st.values() if torch.is_tensor(v) and v.dim() > 0]
        return {"optimizer": moments}
