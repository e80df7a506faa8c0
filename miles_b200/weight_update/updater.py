"""Trainer → rollout weight synchronisation.

Session frame (reference: weight_update/session.py:14-99, updater.py:123-171):
    pause_generation → flush_cache → begin_weight_update → [bucket stream] → end_weight_update
    → update_weight_version → continue_generation
with gloo-style barriers between phases when several trainer ranks take part.

Transfer protocols (`--update-weight-transfer-mode`):
* `alias`   colocated engine built on the trainer's own model object: nothing moves, version bump only.
* `nvlink`  colocated engine with its own buffers in the same layout on the same / a peer GPU: one fused
            kernel per bucket reshards (and, when the engine serves fp8/MXFP8, block-quantises) trainer
            shards straight into the engine's buffers through peer pointers (`fused_weight_sync`).
* `tensor`  bucket stream of HF-named full tensors handed to `engine.update_weights_from_tensor`
            (the CUDA-IPC path of the reference, protocols/cuda_ipc.py:34-264, without serialisation
            because the engine lives in this process).
* `broadcast` HF-named buckets broadcast from trainer rank 0 over a process group that includes remote
            engine processes (reference protocols/broadcast.py:21-208); HTTP engines are told names,
            dtypes and shapes first.
* `disk`    HF safetensors snapshot + `update_weights_from_disk`.
* `delta`   per-version XOR deltas on shared storage written by `weight_update.delta.DeltaWriter`; in-process engines
            follow with a `DeltaReader`, remote ones load the version directory (reference protocols/delta.py:69-470).

Command-line names (`--update-weight-transfer-mode`) map onto these: `broadcast_packed` = `broadcast` with flattened
buckets, `cuda_ipc` = `tensor` (same-process hand-off of device tensors: no handle serialisation is needed), `p2p` =
`nvlink` (peer-memory stores are the point-to-point transfer engine of one NVSwitch box; engines in other processes or on
other boxes are refused with a message that names `broadcast`), `delta` = `delta`.
"""
from __future__ import annotations

import time
from typing import Any

import torch
import torch.distributed as dist

from .hf_iterator import iter_hf_weights


class WeightUpdater:
    def __init__(self, args, actor, engines, mode: str | None = None, quant: str | None = None):
        self.args, self.actor = args, actor
        self.engines = list(engines) if isinstance(engines, (list, tuple)) else [engines]
        mode = mode or getattr(args, "update_weight_transfer_mode", "auto")
        if mode == "auto":
            if all(getattr(e, "model", None) is actor.model for e in self.engines):
                mode = "alias"
            elif all(hasattr(e, "model") for e in self.engines) and actor.device.type == "cuda" and \
                    all(_same_layout(e, actor) or _can_reshard(e, actor) for e in self.engines):
                mode = "nvlink"
            else:
                mode = "tensor"
        self.packed = bool(getattr(args, "broadcast_packed", False))
        if mode not in CLI_MODES:
            raise ValueError(f"unknown weight transfer mode {mode!r}; choose one of {sorted(CLI_MODES)}")
        impl = CLI_MODES[mode]
        if mode == "broadcast_packed":
            self.packed = True
        if mode == "p2p" and not all(hasattr(e, "model") for e in self.engines):
            raise ValueError("--update-weight-transfer-mode p2p writes into the engine's buffers through peer memory and needs "
                             "the engine in this process; use broadcast for engines behind HTTP")
        assert hasattr(self, f"_send_{impl}"), impl
        self.cli_mode = mode
        self.mode = impl
        self.quant = quant or (getattr(args, "export_quant", None) if impl in ("disk", "delta", "broadcast", "tensor") else None)
        if self.quant == "none":
            self.quant = None
        self.framed = False          # True while a controller frames the transfer (it pauses, flushes and resumes the engines)
        self._reshard_plans: dict[int, Any] = {}
        self._delta_writer = None
        self._delta_readers: dict[int, Any] = {}
        self.last_seconds = 0.0
        self.connected_engines_hash = None

    # ---- session frame -------------------------------------------------------------------
    def _is_leader(self) -> bool:
        return not dist.is_initialized() or dist.get_rank() == 0

    def _barrier(self):
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    def update_weights(self) -> dict:
        t0 = time.perf_counter()
        version = self.actor.weight_version
        if not self.framed:
            for e in self.engines:
                e.pause_generation(getattr(self.args, "pause_generation_mode", None) or "retract")
                e.flush_cache()
        self._barrier()
        t1 = time.perf_counter()
        ok = False
        try:
            nbytes = getattr(self, f"_send_{self.mode}")()
            if self.actor.device.type == "cuda":
                torch.cuda.synchronize()
            fab = getattr(getattr(self.actor, "ps", None), "fabric", None)
            if fab is not None:
                fab.check()
            ok = True
        finally:
            # a failed transfer must not leave the engines paused: they resume on the version they hold
            if not ok and not self.framed:
                for e in self.engines:
                    e.continue_generation()
        self._barrier()
        t2 = time.perf_counter()
        if not self.framed:
            for e in self.engines:
                e.update_weight_version(version)
                e.continue_generation()
        if getattr(self.args, "ci_test", False) and not self.framed:
            for e in self.engines:
                assert e.get_weight_version() == version, "engine weight version differs from the trainer's"
        if getattr(self.args, "check_weight_update_equal", False):
            self.check_equal()
        self.last_seconds = t2 - t1
        return {"mode": self.mode, "bytes": nbytes, "seconds": t2 - t1, "total_seconds": time.perf_counter() - t0,
                "weight_version": version}

    # ---- protocols -----------------------------------------------------------------------
    def _send_alias(self) -> int:
        n = 0
        for e in self.engines:                         # engines that serve MXFP8 copies of the shared bf16 weights
            if getattr(e, "quant_buffers", None):
                from ..parallel import weight_sync

                n += weight_sync.fused_weight_sync(self.actor, e, quant="mxfp8")
        return n

    def _send_nvlink(self) -> int:
        from ..parallel import weight_sync

        n = 0
        for i, e in enumerate(self.engines):
            if _same_layout(e, self.actor):
                n += weight_sync.fused_weight_sync(self.actor, e, quant=self.quant)
                continue
            # different TP / EP layout: every trainer rank stores the rectangles of its shards straight into the shards of
            # every engine rank (peer memory), one kernel per transfer, no gathered full tensors
            assert _can_reshard(e, self.actor), "resharding sync needs the NVLink fabric and an in-process engine on every rank"
            plan = self._reshard_plans.get(i)
            if plan is None:
                from ..parallel.reshard import ReshardPlan

                plan = self._reshard_plans[i] = ReshardPlan(self.actor, e, self.actor.ps.fabric, quant=self.quant)
            n += plan.run()
        return n

    def _send_tensor(self) -> int:
        n = 0
        size = getattr(self.args, "update_weight_buffer_size", 512 << 20)
        for bucket in iter_hf_weights(self.actor, bucket_bytes=size, quant=self.quant):
            n += sum(t.numel() * t.element_size() for _, t in bucket)
            for e in self.engines:
                e.update_weights_from_tensor(bucket, load_format="flattened_bucket")
        return n

    def _send_broadcast(self) -> int:
        from .broadcast import broadcast_buckets

        return broadcast_buckets(self)

    def _send_disk(self) -> int:
        import os
        import tempfile

        from ..checkpoint import hf_io

        d = getattr(self.args, "update_weight_disk_dir", None) or tempfile.mkdtemp(prefix="miles_sync_")
        d = os.path.join(d, f"v{self.actor.weight_version}")
        from .quantize import hf_quant_config

        hf_io.save_hf_sharded(d, iter_hf_weights(self.actor, bucket_bytes=None, quant=self.quant), self.actor.cfg,
                              write=self._is_leader(), extra_config=hf_quant_config(self.quant) if self.quant else None)
        self._barrier()
        for e in self.engines:
            e.update_weights_from_disk(d)
        return sum(p.numel() * p.element_size() for p in self.actor.model.parameters())

    def _send_delta(self) -> int:
        import os
        import tempfile

        from .delta import DeltaReader, DeltaWriter

        root = getattr(self.args, "update_weight_disk_dir", None) or getattr(self, "_delta_root", None)
        if root is None:
            root = self._delta_root = tempfile.mkdtemp(prefix="miles_delta_")
        version = self.actor.weight_version
        named = ((n, t) for bucket in iter_hf_weights(self.actor, bucket_bytes=None, quant=self.quant) for n, t in bucket)
        nbytes = 0
        if self._is_leader():
            if self._delta_writer is None:
                self._delta_writer = DeltaWriter(root, full_every=getattr(self.args, "update_weight_delta_full_every", 10))
            nbytes = self._delta_writer.publish(version, named).get("stored_bytes", 0)
        else:
            for _ in named:           # the shard gathers inside the iterator are collective
                pass
        self._barrier()
        for i, e in enumerate(self.engines):
            if hasattr(e, "model"):
                rd = self._delta_readers.setdefault(i, DeltaReader(root))
                e.update_weights_from_tensor(list(rd.update_to(version).items()))
            else:
                e.update_weights_from_disk(os.path.join(root, f"v{version}"))
        return nbytes

    # ---- verification --------------------------------------------------------------------
    def check_equal(self):
        """Engine-side tensor compare (`--check-weight-update-equal`)."""
        for e in self.engines:
            if not hasattr(e, "model"):
                continue
            mine = dict(self.actor.model.named_parameters())
            skip = list(getattr(self.args, "check_weight_update_skip_list", None) or [])
            quant_ok = bool(getattr(self.args, "check_weight_update_allow_quant_error", False)) and self.quant
            for n, p in e.model.named_parameters():
                if n not in mine or any(pat in n for pat in skip):
                    continue
                if quant_ok:
                    # block-quantised transfer: values agree to the quantiser's step (2^-3 relative for e4m3 mantissas)
                    a, b = p.data.float(), mine[n].data.float()
                    if not torch.allclose(a, b, rtol=0.07, atol=1e-3 * float(b.abs().max())):
                        raise AssertionError(f"weight {n} differs beyond quantisation error after update")
                elif not torch.equal(p.data, mine[n].data):
                    raise AssertionError(f"weight {n} differs between trainer and engine after update")


# command-line name → protocol implemented here
CLI_MODES = {"alias": "alias", "nvlink": "nvlink", "tensor": "tensor", "broadcast": "broadcast", "disk": "disk", "delta": "delta",
             "broadcast_packed": "broadcast", "cuda_ipc": "tensor", "p2p": "nvlink"}


def _can_reshard(engine, actor) -> bool:
    ps = getattr(actor, "ps", None)
    return (ps is not None and getattr(ps, "fabric", None) is not None and hasattr(engine, "model")
            and engine.model is not actor.model and ps.pp_size == 1 and getattr(engine.ps, "pp_size", 1) == 1)


def _same_layout(engine, actor) -> bool:
    a, b = engine.ps, actor.ps
    return (a.tp_size, a.ep_size, a.pp_size, a.tp_rank, a.ep_rank, a.pp_rank) == \
           (b.tp_size, b.ep_size, b.pp_size, b.tp_rank, b.ep_rank, b.pp_rank)
