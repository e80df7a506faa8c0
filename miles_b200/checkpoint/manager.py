"""Checkpoint save / load for the trainer.

Directory layout is the reference's (miles/backends/megatron_utils/checkpoint.py:12-14,107-299;
tracker miles/backends/training_utils/checkpoint/tracker.py:5-19):

    <save>/latest_checkpointed_iteration.txt
    <save>/iter_{N:07d}/.metadata, __R_0.distcp, common.pt   --ckpt-format torch_dist (default): Megatron-named entries,
                                                        chunks written by their owners, optimizer state in model space
                                                        (checkpoint/sharded.py); reloadable under any parallel layout
    <save>/iter_{N:07d}/model_rank{R:05d}.pt            --ckpt-format native: this rank's shards by our names
    <save>/iter_{N:07d}/optim_rank{R:05d}.pt            … its optimizer shard + scheduler
    <save>/iter_{N:07d}/hf/…                            optional HF safetensors export (--save-hf)
    <save>/iter_{N:07d}/.complete                       written last, after every rank finished
    <save>/rollout/global_dataset_state_dict_{N}.pt     data-source state (written by the data source)

Loading accepts (a) such a directory (`--load`), (b) an HF directory (`--hf-checkpoint` / `--ref-load`),
(c) a Megatron `torch_dist` directory through `miles_b200.checkpoint.torch_dist`.
The collective write protocol — every rank reports success or its error string, all ranks raise if any
failed, the completion marker appears only after a barrier — follows checkpoint/io.py:18-81.
"""
from __future__ import annotations

import os
import shutil
from typing import Any

import torch
import torch.distributed as dist

from ..models.convert import hf_state_to_ours, load_named_into_model
from . import hf_io
from ..weight_update.quantize import hf_quant_config

TRACKER = "latest_checkpointed_iteration.txt"


def iter_dir(root: str, iteration: int) -> str:
    return os.path.join(root, f"iter_{iteration:07d}")


def read_tracker(root: str) -> int | str | None:
    path = os.path.join(root, TRACKER)
    if not os.path.exists(path):
        return None
    txt = open(path).read().strip()
    return "release" if txt == "release" else int(txt)


def write_tracker(root: str, iteration: int | str):
    tmp = os.path.join(root, f".{TRACKER}.tmp")
    with open(tmp, "w") as f:
        f.write(str(iteration))
    os.replace(tmp, os.path.join(root, TRACKER))


def _rank_world():
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def collective_write(directory: str, write_fn, group=None) -> None:
    """Run `write_fn(directory)` on every rank; raise everywhere if anyone failed; mark complete."""
    rank, world = _rank_world()
    os.makedirs(directory, exist_ok=True)
    err = None
    try:
        write_fn(directory)
    except Exception as e:  # collected and re-raised on every rank
        err = f"rank {rank}: {type(e).__name__}: {e}"
    if world > 1:
        errs: list = [None] * world
        dist.all_gather_object(errs, err, group=group)
    else:
        errs = [err]
    bad = [e for e in errs if e]
    if bad:
        raise RuntimeError("checkpoint write failed: " + "; ".join(bad))
    if rank == 0:
        open(os.path.join(directory, ".complete"), "w").close()
    if world > 1:
        dist.barrier(group=group)


class _AsyncSave:
    """`--async-save`: the training thread stages this rank's chunks in host memory, a writer thread plans and writes the
    store over its OWN gloo process group (so its collectives never interleave with the trainer's), then marks the
    directory complete and moves the tracker.  At most one save is in flight: the next save, `finalize_async_save()` and
    interpreter exit wait for it and re-raise its error (the reference: `--async-save`,
    miles/backends/megatron_utils/checkpoint.py, Megatron's async strategy)."""

    def __init__(self):
        self.thread = None
        self.error: BaseException | None = None
        self.group = None

    def ensure_group(self):
        if self.group is None and dist.is_initialized() and dist.get_world_size() > 1:
            self.group = dist.new_group(backend="gloo")              # collective: every rank takes this path together
        return self.group

    def wait(self):
        t, self.thread = self.thread, None
        if t is not None:
            t.join()
        if self.error is not None:
            e, self.error = self.error, None
            raise RuntimeError(f"asynchronous checkpoint save failed: {e}") from e

    def start(self, fn):
        import threading

        self.wait()

        def run():
            try:
                fn()
            except BaseException as e:  # surfaced by the next wait()
                self.error = e

        self.thread = threading.Thread(target=run, name="ckpt-writer", daemon=False)
        self.thread.start()


_ASYNC = _AsyncSave()


def finalize_async_save():
    """Block until the checkpoint in flight (if any) is on disk; raises if it failed."""
    _ASYNC.wait()


def _export_quant(args):
    q = getattr(args, "export_quant", None)
    return None if q in (None, "none") else q


def save_from_actor(actor, args, iteration: int, with_optimizer: bool = True):
    root = args.save
    assert root, "--save is required to save checkpoints"
    rank, world = _rank_world()
    d = iter_dir(root, iteration)

    fmt = getattr(args, "ckpt_format", "torch_dist")
    from . import sharded

    use_dist = (fmt == "torch_dist" and not getattr(actor, "fsdp", False) and sharded.supported(actor.cfg, actor.ps)
                and hasattr(actor.model, "named_parameters_global"))
    with_opt = with_optimizer and not getattr(args, "no_save_optim", False)

    def write_dist(directory):
        meta = {"iteration": iteration, "cfg": actor.cfg.asdict(), "world_size": world, "checkpoint_version": 3.0,
                "weight_version": actor.weight_version, "global_step": actor.global_step,
                "optimizer": {"step_count": actor.optimizer.step_count}, "scheduler": actor.scheduler.state_dict(),
                "args": {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, type(None), list, tuple))}}
        sharded.save(actor, directory, with_optimizer=with_opt, common=meta)
        torch.save({"rng": torch.get_rng_state()}, os.path.join(directory, f"rng_rank{rank:05d}.pt"))
        _save_hf(directory)

    def _save_hf(directory):
        if getattr(args, "save_hf", False):
            from ..weight_update.hf_iterator import iter_hf_weights

            hf_io.save_hf_sharded(os.path.join(directory, "hf"), iter_hf_weights(actor, bucket_bytes=None, quant=_export_quant(args)), actor.cfg,
                                  write=(rank == 0), src_dir=getattr(args, "hf_checkpoint", None),
                                  extra_config=hf_quant_config(_export_quant(args)) if _export_quant(args) else None)

    def write(directory):
        state = {n: t.detach().cpu() for n, t in actor.named_weights()}       # model-wide names (pipeline stages too)
        meta = {"iteration": iteration, "cfg": actor.cfg.asdict(), "world_size": world,
                "tp": actor.ps.tp_size, "pp": actor.ps.pp_size, "ep": actor.ps.ep_size,
                "tp_rank": actor.ps.tp_rank, "pp_rank": actor.ps.pp_rank, "ep_rank": actor.ps.ep_rank,
                "dp_rank": actor.ps.dp_rank, "weight_version": actor.weight_version, "global_step": actor.global_step}
        torch.save({"model": state, "meta": meta}, os.path.join(directory, f"model_rank{rank:05d}.pt"))
        if with_opt:
            torch.save({"optimizer": actor.optimizer.state_dict(), "scheduler": actor.scheduler.state_dict(),
                        "rng": torch.get_rng_state()}, os.path.join(directory, f"optim_rank{rank:05d}.pt"))
        _save_hf(directory)

    def write_fsdp(directory):
        from . import fsdp_dcp

        fsdp_dcp.save(actor, directory, iteration, with_optimizer=with_opt)
        _save_hf(directory)

    if use_dist and getattr(args, "async_save", False):
        group = _ASYNC.ensure_group()
        _ASYNC.wait()
        staged = sharded.stage(actor, with_optimizer=with_opt, to_host=True)
        meta = {"iteration": iteration, "cfg": actor.cfg.asdict(), "world_size": world, "checkpoint_version": 3.0,
                "weight_version": actor.weight_version, "global_step": actor.global_step,
                "optimizer": {"step_count": actor.optimizer.step_count}, "scheduler": actor.scheduler.state_dict()}
        rng = torch.get_rng_state()

        def job():
            def w(directory):
                sharded.write_staged(staged, directory, common=meta, process_group=group)
                torch.save({"rng": rng}, os.path.join(directory, f"rng_rank{rank:05d}.pt"))

            collective_write(d, w, group=group)
            if rank == 0:
                write_tracker(root, iteration)

        _ASYNC.start(job)
        return
    if fmt == "torch_dist" and getattr(actor, "fsdp", False):
        collective_write(d, write_fsdp)
    else:
        collective_write(d, write_dist if use_dist else write)
    if rank == 0:
        write_tracker(root, iteration)


def load_weights_only(actor, path: str):
    """HF dir, this package's iter dir / root, or Megatron torch_dist dir → model weights."""
    if os.path.exists(os.path.join(path, "model.safetensors.index.json")) or \
            any(f.endswith(".safetensors") for f in os.listdir(path)):
        hf = hf_io.load_hf_dir(path)
        load_named_into_model(actor.model, hf_state_to_ours(hf, actor.cfg).items(), actor.cfg, actor.ps)
        return None
    it = read_tracker(path)
    d = path
    if it is not None:
        d = os.path.join(path, "release") if it == "release" else iter_dir(path, it)
    rank, _ = _rank_world()
    mine = os.path.join(d, f"model_rank{rank:05d}.pt")
    if os.path.exists(mine):
        blob = torch.load(mine, map_location="cpu", weights_only=False)
        load_named_into_model(actor.model, blob["model"].items(), actor.cfg, actor.ps)
        return blob["meta"]
    from . import fsdp_dcp, torch_dist

    if fsdp_dcp.is_fsdp_dir(d):
        assert getattr(actor, "fsdp", False), f"{d} holds an FSDP-backend checkpoint; load it with --train-backend fsdp"
        meta = fsdp_dcp.load_model(actor, d)
        return {"iteration": meta.get("iteration", 0), "weight_version": meta.get("weight_version", 0),
                "global_step": meta.get("global_step", 0), "optimizer": {"step_count": meta.get("optimizer_steps", 0)}}
    if torch_dist.is_torch_dist_dir(d):
        from ..models.convert import megatron_to_ours
        from . import sharded

        if sharded.supported(actor.cfg, actor.ps) and hasattr(actor.model, "named_parameters_global") and \
                not getattr(actor, "fsdp", False) and torch_dist.has_per_layer_names(d):
            common = sharded.load(actor, d, with_optimizer=False)
            return common or {"iteration": it if isinstance(it, int) else 0}
        full = megatron_to_ours(torch_dist.load_state(d), actor.cfg)
        load_named_into_model(actor.model, full.items(), actor.cfg, actor.ps)
        return {"iteration": it if isinstance(it, int) else 0}
    raise FileNotFoundError(f"no loadable checkpoint under {path}")


def load_into_actor(actor, args) -> int | None:
    """Resume from --load if it has a tracker; else initialise from --hf-checkpoint. Returns the iteration."""
    load = getattr(args, "load", None)
    if load and os.path.isdir(load) and read_tracker(load) is not None:
        meta = load_weights_only(actor, load)
        it = read_tracker(load)
        actor.optimizer.reload_master_from_params()
        rank, _ = _rank_world()
        d = iter_dir(load, it) if isinstance(it, int) else os.path.join(load, "release")
        opt_path = os.path.join(d, f"optim_rank{rank:05d}.pt")
        want_opt = not getattr(args, "no_load_optim", False) and not getattr(args, "finetune", False)
        from . import fsdp_dcp, sharded, torch_dist

        if want_opt and fsdp_dcp.is_fsdp_dir(d) and getattr(actor, "fsdp", False):
            if fsdp_dcp.load_optimizer(actor, d, load_rng=not getattr(args, "no_load_rng", False)) and meta:
                actor.optimizer.step_count = meta.get("optimizer", {}).get("step_count", 0)
        elif want_opt and not os.path.exists(opt_path) and torch_dist.is_torch_dist_dir(d) and sharded.has_optimizer(d) \
                and hasattr(actor.optimizer, "domains"):
            sharded.load_optimizer(actor, d)
            if meta and "scheduler" in meta:
                actor.scheduler.load_state_dict(meta["scheduler"])
                actor.optimizer.step_count = meta.get("optimizer", {}).get("step_count", 0)
            rng = os.path.join(d, f"rng_rank{rank:05d}.pt")
            if os.path.exists(rng) and not getattr(args, "no_load_rng", False):
                torch.set_rng_state(torch.load(rng, weights_only=False)["rng"])
        elif os.path.exists(opt_path) and want_opt:
            blob = torch.load(opt_path, map_location="cpu", weights_only=False)
            actor.optimizer.load_state_dict(blob["optimizer"])
            actor.scheduler.load_state_dict(blob["scheduler"])
        if meta:
            actor.weight_version = meta.get("weight_version", 0)
            actor.global_step = meta.get("global_step", 0)
        if getattr(args, "finetune", False) or it == "release":
            return None
        return int(it)
    hf = getattr(args, "hf_checkpoint", None)
    if hf and os.path.isdir(hf) and any(f.endswith(".safetensors") for f in os.listdir(hf)):
        load_weights_only(actor, hf)
        actor.optimizer.reload_master_from_params()
    return None


def cleanup_old(root: str, keep_last: int):
    its = sorted(int(d.split("_")[1]) for d in os.listdir(root) if d.startswith("iter_") and
                 os.path.exists(os.path.join(root, d, ".complete")))
    for it in its[:-keep_last]:
        shutil.rmtree(iter_dir(root, it), ignore_errors=True)
