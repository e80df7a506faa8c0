"""Checkpoints of the FSDP backend as DCP stores, one per kind of state.

The reference's FSDP backend writes `iter_XXXXXXX/{model,optimizer,lr_scheduler}/` — three DCP stores whose entries are
the sharded (DTensor) parameters under `model_state.model.<name>`, the AdamW state under
`optim_state.optim.state.<name>.{exp_avg,exp_avg_sq,step}` and the scheduler state — plus `rng.pt` and `meta.json`, so
that weights load without the optimizer and a run resumes on another number of ranks
(miles/backends/fsdp_utils/checkpoint.py:20-60, 96-160, 196-250).  The same directory layout is written here straight
from the `fully_shard` DTensors: DCP stores each rank's shard as a chunk and re-slices on load, whatever the new world
size.  Entry names are this package's parameter names.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist


def _model_state(actor) -> dict:
    return {"model_state": {"model": {n: p for n, p in actor.model.named_parameters()}}}


def _ensure_moments(opt):
    if not opt.opt.state:                            # AdamW creates its state lazily: one step with zero gradients, lr 0
        for p in opt.params:
            p.grad = torch.zeros_like(p)
        for g in opt.opt.param_groups:
            g["lr"] = 0.0
        opt.opt.step()
        opt.zero_grad()
        for st in opt.opt.state.values():
            st["step"].zero_()


def _optim_state(actor) -> dict:
    opt = actor.optimizer
    state = {}
    for n, p in opt.named:
        st = opt.opt.state.get(p)
        if st:
            state[n] = {k: v for k, v in st.items() if torch.is_tensor(v)}
    groups = [{k: v for k, v in g.items() if k != "params"} for g in opt.opt.param_groups]
    return {"optim_state": {"optim": {"state": state, "param_groups": groups}}}


def is_fsdp_dir(d: str) -> bool:
    return os.path.exists(os.path.join(d, "model", ".metadata"))


def save(actor, directory: str, iteration: int, with_optimizer: bool = True) -> None:
    import torch.distributed.checkpoint as dcp

    rank = dist.get_rank() if dist.is_initialized() else 0
    for sub in ("model", "optimizer", "lr_scheduler"):
        os.makedirs(os.path.join(directory, sub), exist_ok=True)
    dcp.save(_model_state(actor), checkpoint_id=os.path.join(directory, "model"))
    if with_optimizer:
        dcp.save(_optim_state(actor), checkpoint_id=os.path.join(directory, "optimizer"))
        dcp.save({"lr_scheduler_state": {"lr_scheduler": dict(actor.scheduler.state_dict())}},
                 checkpoint_id=os.path.join(directory, "lr_scheduler"))
    if rank == 0:
        rng = {"torch": torch.get_rng_state()}
        if torch.cuda.is_available():
            rng["cuda"] = torch.cuda.get_rng_state_all()
        torch.save(rng, os.path.join(directory, "rng.pt"))
        meta = {"iteration": iteration, "rollout_id": iteration, "next_rollout_id": iteration + 1,
                "global_step": actor.global_step, "weight_version": actor.weight_version,
                "optimizer_steps": actor.optimizer.step_count,
                "world_size": dist.get_world_size() if dist.is_initialized() else 1, "timestamp": time.time()}
        with open(os.path.join(directory, "meta.json"), "w") as f:
            json.dump(meta, f)


def load_model(actor, directory: str) -> dict:
    import torch.distributed.checkpoint as dcp

    dcp.load(_model_state(actor), checkpoint_id=os.path.join(directory, "model"))
    path = os.path.join(directory, "meta.json")
    return json.load(open(path)) if os.path.exists(path) else {}


def load_optimizer(actor, directory: str, load_rng: bool = True) -> bool:
    import torch.distributed.checkpoint as dcp

    if not os.path.exists(os.path.join(directory, "optimizer", ".metadata")):
        return False
    _ensure_moments(actor.optimizer)
    st = _optim_state(actor)
    dcp.load(st, checkpoint_id=os.path.join(directory, "optimizer"))
    for g, saved in zip(actor.optimizer.opt.param_groups, st["optim_state"]["optim"]["param_groups"]):
        g.update({k: v for k, v in saved.items() if k != "params"})
    if os.path.exists(os.path.join(directory, "lr_scheduler", ".metadata")):
        sd = {"lr_scheduler_state": {"lr_scheduler": dict(actor.scheduler.state_dict())}}
        dcp.load(sd, checkpoint_id=os.path.join(directory, "lr_scheduler"))
        actor.scheduler.load_state_dict(sd["lr_scheduler_state"]["lr_scheduler"])
    rng = os.path.join(directory, "rng.pt")
    if load_rng and os.path.exists(rng):
        torch.set_rng_state(torch.load(rng, weights_only=False)["torch"])
    return True
