"""Trainer worker: owns one rank's model shard, optimizer shard and weight tags.

The worker contract is the reference's `TrainRayActor` (miles/ray/train_actor.py:56-243;
Megatron subclass miles/backends/megatron_utils/actor.py:105-1008): `init`, `train`,
`update_weights`, `save_model`, `sleep`, `wake_up`, plus log-prob-only passes for the reference
and old-actor tags.  One RL step (reference call stack: actor.py:657-812 → model.py:281-872):

    shard of rollout data → micro-batches → [ref log-probs] → [old log-probs] → advantages
    → for each optimizer step: forward/backward over micro-batches → grad reduce → Adam
"""
from __future__ import annotations

import os
import time
from argparse import Namespace
from contextlib import contextmanager
from typing import Any

import torch
import torch.distributed as dist

from ..args import model_config_from_args
from ..models.config import ModelConfig
from ..models.qwen3 import ForwardMeta, Qwen3Model, build_model
from ..parallel.state import ParallelState
from ..utils.timer import Timer
from . import math_utils as mu
from .advantages import compute_advantages_and_returns
from .data import PackedBatch, flat_per_token, make_micro_batches, pack_micro_batch
from .losses import LossBatch, loss_function
from .optimizer import DistributedAdam, LRScheduler, mark_expert_params


class TensorBackuper:
    """Named snapshots of the model weights in pinned host memory (`actor`, `ref`, `old_actor`,
    `teacher`), swapped into the live parameters for log-prob passes
    (reference: weights_backuper in miles/backends/megatron_utils/actor.py:418-434,787-790)."""

    def __init__(self, model: torch.nn.Module):
        self.model = model
        self.tags: dict[str, dict[str, torch.Tensor]] = {}

    def backup(self, tag: str):
        store = self.tags.setdefault(tag, {})
        from .fsdp import local_data

        for n, p in self.model.named_parameters():
            src = local_data(p)                 # the shard of an FSDP parameter, the tensor itself otherwise
            if n not in store:
                t = torch.empty(src.shape, dtype=src.dtype, device="cpu")
                if torch.cuda.is_available():
                    t = t.pin_memory()
                store[n] = t
            store[n].copy_(src, non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    def restore(self, tag: str):
        from .fsdp import local_data

        store = self.tags[tag]
        for n, p in self.model.named_parameters():
            local_data(p).copy_(store[n], non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    def has(self, tag: str) -> bool:
        return tag in self.tags


class TrainActor:
    def __init__(self, args: Namespace, ps: ParallelState | None = None, device: str | torch.device | None = None,
                 role: str = "actor"):
        self.args = args
        self.ps = ps or ParallelState.single()
        self.role = role
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.timer = Timer()
        self.model: Qwen3Model | None = None
        self.optimizer: DistributedAdam | None = None
        self.cfg: ModelConfig | None = None
        self.asleep = False
        self.weight_version = 0
        self.global_step = 0
        self.start_rollout_id = 0

    # ---------------------------------------------------------------------------------------
    # init
    # ---------------------------------------------------------------------------------------
    def init(self, cfg: ModelConfig | None = None, with_ref: bool | None = None) -> int:
        args = self.args
        self.cfg = cfg or model_config_from_args(args)
        dtype = torch.float32 if getattr(args, "fp32", False) or not getattr(args, "bf16", True) else torch.bfloat16
        torch.manual_seed(args.seed)
        if getattr(args, "fp8_recipe", None) == "mxfp8" and self.device.type == "cuda":
            from ..ops import cuda as _cuda_ops

            _cuda_ops.MXFP8_LINEAR = True       # projections run their forward on the block-scaled MXFP8 tensor-core path
            if getattr(args, "fp8_backward", False):
                _cuda_ops.MXFP8_BACKWARD = True  # and both gradient products, on operands quantised along the contraction axis
        self.fsdp = getattr(args, "train_backend", "native") == "fsdp" and dist.is_initialized() and dist.get_world_size() > 1
        compute_dtype = self.compute_dtype = dtype
        if self.fsdp:
            dtype = torch.float32               # FSDP keeps fp32 shards (the master weights) and computes in `compute_dtype`
        provider = getattr(args, "custom_model_provider_path", None)
        if provider:
            from ..utils.misc import load_function
            self.model = load_function(provider)(args, self.cfg, self.ps, dtype, self.device)
        else:
            self.model = build_model(self.cfg, self.ps, dtype=dtype, device=self.device, seed=args.seed)
        if getattr(args, "lora_rank", 0) > 0:
            from .lora import apply_lora
            apply_lora(self.model, args)
        if self.role == "critic":
            from .critic import attach_value_head
            attach_value_head(self.model, self.cfg, dtype, self.device)
        mark_expert_params(self.model)
        lr0 = args.lr if self.role == "actor" else args.critic_lr
        if self.fsdp:
            # parameters sharded per decoder layer (PyTorch FSDP2), AdamW on the shards; see train/fsdp.py
            from .fsdp import FsdpOptimizer, shard_model

            shard_model(self.model, self.ps, self.device, dp_replicate=getattr(args, "fsdp_dp_replicate", 1),
                        compute_dtype=compute_dtype)
        named = [(n, p) for n, p in self.model.named_parameters() if p.requires_grad]   # LoRA / critic freeze the rest
        if self.fsdp:
            self.optimizer = FsdpOptimizer(named, lr=lr0, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                                           weight_decay=args.weight_decay, clip_grad=args.clip_grad)
        else:
            # --offload-train: optimizer state lives in a VMM arena; sleep() releases its physical pages (contents kept in
            # pinned host memory), wake_up() maps them back at the same addresses
            self.arena = None
            state_alloc = None
            if getattr(args, "offload_train", False) and getattr(args, "offload_train_mode", "vmm") == "vmm":
                from ..utils.memory import make_arena

                self.arena = make_arena(self.device)
                if self.arena is not None:
                    state_alloc = lambda n, dt, dev, tag: self.arena.empty((n,), dt, tag="optimizer")  # noqa: E731
            self.optimizer = DistributedAdam(
                named, lr=lr0, betas=(args.adam_beta1, args.adam_beta2),
                eps=args.adam_eps, weight_decay=args.weight_decay, clip_grad=args.clip_grad, ps=self.ps,
                allocator=self._symmetric_allocator(), state_allocator=state_alloc,
                nvme_dir=self._nvme_dir(), nvme_bucket_numel=int(getattr(args, "optimizer_nvme_bucket_numel", 64 << 20) or (64 << 20)))
        self.tp_replicated = {n for n, p in named if _tp_replicated(n)}
        if self.ps.tp_size > 1:
            self.optimizer.mark_tp_replicated(self.tp_replicated, named)
        self.scheduler = LRScheduler(self.optimizer.lr, args.min_lr, args.lr_warmup_iters, args.lr_decay_iters,
                                     args.lr_decay_style)
        from ..utils.profiling import TrainProfiler

        self.profiler = TrainProfiler(args)
        self.profiler.on_init_end()
        self.backuper = TensorBackuper(self.model)
        if getattr(args, "use_miles_dashboard", False) and getattr(args, "dump_details", None):
            from ..dashboard.phases import PhaseSink

            self.phase_sink = PhaseSink(args.dump_details, self.ps.rank, self.role)
            self.timer.sinks.append(self.phase_sink)          # every timed span of this rank becomes a lane interval
        from ..utils.dumper import DumperSwitch

        self.dumper = DumperSwitch.from_args(args, self.ps.rank)       # --dumper-enable + per-phase lists; None when off
        if self.dumper is not None:
            self.dumper.register(self.model)
        self.indep_dp = self._make_indep_dp()
        # checkpoints
        from ..checkpoint import manager as ckpt
        loaded_iter = ckpt.load_into_actor(self, args)
        if loaded_iter is not None:
            self.start_rollout_id = loaded_iter + 1
            if getattr(args, "reset_optimizer_states", False):
                self.optimizer.reset_state()           # keep the weights, restart Adam (a new task on an old checkpoint)
            if getattr(args, "rematerialize_param_from_master_weight", False) or getattr(args, "check_rematerialize_param_from_master_weight", False):
                self._rematerialize(check=getattr(args, "check_rematerialize_param_from_master_weight", False))
        if getattr(args, "start_rollout_id", None) is not None:
            self.start_rollout_id = int(args.start_rollout_id)
        need_ref = getattr(args, "need_ref", False) if with_ref is None else with_ref
        if need_ref and self.role == "actor":
            if getattr(args, "ref_load", None) and args.ref_load != getattr(args, "hf_checkpoint", None):
                self.backuper.backup("actor")
                ckpt.load_weights_only(self, args.ref_load)
                self.backuper.backup("ref")
                self.backuper.restore("actor")
            else:
                self.backuper.backup("ref")
        if self.role == "actor" and getattr(args, "use_opd", False) and getattr(args, "opd_type", None) == "megatron":
            load = getattr(args, "opd_teacher_load", None)
            assert load, "--opd-type megatron needs --opd-teacher-load"
            step = getattr(args, "opd_teacher_ckpt_step", None)
            if step is not None:                      # a chosen iteration instead of the tracker's latest
                load = ckpt.iter_dir(load, int(step))
            self.backuper.backup("actor")
            ckpt.load_weights_only(self, load)
            self.backuper.backup("teacher")
            self.backuper.restore("actor")
        return self.start_rollout_id

    def _rematerialize(self, check: bool = False):
        """Rewrite the compute-dtype parameters of this rank's optimizer shards from the fp32 master copy (a checkpoint's
        bf16 weights and master weights can disagree by one rounding after a dtype or layout change); with `check` the
        rewrite must be a no-op (reference: megatron_utils/rematerialize_utils.py)."""
        opt = self.optimizer
        for d in getattr(opt, "domains", []):
            lo, hi = d.shard
            fresh = d.master.to(d.param_buf.dtype)
            if check and not torch.equal(fresh, d.param_buf[lo:hi]):
                bad = (fresh != d.param_buf[lo:hi]).sum().item()
                raise AssertionError(f"{d.name}: {bad} parameters differ from their fp32 master copy")
            d.param_buf[lo:hi].copy_(fresh)
        if hasattr(opt, "_all_gather"):
            for d in opt.domains:
                opt._all_gather(d)

    def _hook(self, flag: str, *a):
        path = getattr(self.args, flag, None)
        if path:
            from ..utils.misc import load_function

            load_function(path)(self.args, self, *a)

    def _make_indep_dp(self):
        """`--indep-dp`: this training world is one cell of several; gradients are averaged across the cells through a
        group that survives the loss of a cell (ft/indep_dp.py).  Rank r of every cell forms one cross-cell group."""
        args = self.args
        n_cells = getattr(args, "indep_dp_num_cells", 1)
        if not getattr(args, "indep_dp", False) or n_cells <= 1:
            return None
        from ..ft.indep_dp import IndepDP

        host, port = args.indep_dp_store.rsplit(":", 1)
        rank = dist.get_rank() if dist.is_initialized() else 0
        cell = args.indep_dp_cell_id
        idp = IndepDP(cell, host, int(port) + rank, backend="nccl" if self.device.type == "cuda" else "gloo",
                      timeout_s=getattr(args, "indep_dp_timeout", 30.0), is_store_master=cell == 0, expected_cells=n_cells)
        if cell == 0:
            idp.members.publish(0, list(range(n_cells)))
        idp.follow_membership()
        return idp

    def _exchange_across_cells(self) -> bool:
        """Average the gradient buffers over the live cells; False when the cells agreed to discard this step."""
        if self.indep_dp is None:
            return True
        buckets = [d.grad_buf for d in self.optimizer.domains]
        finite = all(bool(torch.isfinite(b).all()) for b in buckets)
        committed, cells = self.indep_dp.step(buckets, local_ok=finite)
        self.last_cells = cells
        return committed

    def _symmetric_allocator(self):
        """Flat param/grad buffers come from the fabric's symmetric heap so peers can address them."""
        fab = self.ps.fabric
        if fab is None:
            return None
        return lambda n, dtype, device, tag: fab.alloc(n, dtype, tag=tag)

    # ---------------------------------------------------------------------------------------
    # forward helpers
    # ---------------------------------------------------------------------------------------
    def _meta(self, pb: PackedBatch, replay: bool) -> ForwardMeta:
        rec = getattr(self.args, "recompute_granularity", None) == "full"
        return ForwardMeta(positions=pb.positions, cu_seqlens=pb.cu_seqlens, max_seqlen=pb.max_seqlen,
                           replay_topk=pb.replay_topk if replay else None, recompute=rec)

    def _forward_logprobs(self, pb: PackedBatch, with_entropy: bool, replay: bool):
        if self.ps.cp_size > 1:
            return self._forward_logprobs_cp(pb, with_entropy, replay)
        # vision-language policies take the images of the packed samples next to the token stream
        hidden = (self.model(pb.tokens, self._meta(pb, replay), **pb.mm_inputs) if pb.mm_inputs
                  else self.model(pb.tokens, self._meta(pb, replay)))
        if self.role == "critic":
            h = self.ps.sp_gather(hidden)
            return self.model.value_head(h[pb.gather_index].float()).squeeze(-1), None
        h = self.ps.sp_gather(hidden)[pb.gather_index]
        temp = getattr(self.args, "rollout_temperature", 1.0)
        return self.ps.vocab_parallel_logprob(h, self.model.head_weight(), pb.targets, temp, with_entropy,
                                              self.cfg.vocab_size)

    def _pipe(self):
        if getattr(self, "_pipe_stage", None) is None:
            from ..parallel.pp import PipeStage

            assert self.ps.cp_size == 1, "pipeline + context parallelism is not wired in this trainer"
            self._pipe_stage = PipeStage(self.ps, self.cfg.hidden_size, next(self.model.parameters()).dtype, self.device)
        return self._pipe_stage

    def _forward_logprobs_pp(self, pb: PackedBatch, with_entropy: bool, replay: bool):
        """One micro-batch through this pipeline stage.  Returns (log-probs | values, entropy, StageIO); the first two
        are None except on the last stage."""
        from ..parallel.pp import StageIO

        stage = self._pipe()
        grad = torch.is_grad_enabled()
        hidden_in = stage.recv_forward(pb.tokens.numel(), requires_grad=grad)
        hidden = self.model(pb.tokens, self._meta(pb, replay), hidden_in=hidden_in)
        if not stage.is_last:
            stage.send_forward(hidden)
            return None, None, StageIO(hidden_in, hidden if grad else None)
        lp, ent = self._score_hidden(pb, hidden, with_entropy)
        return lp, ent, StageIO(hidden_in, None)

    def _score_hidden(self, pb: PackedBatch, hidden: torch.Tensor, with_entropy: bool):
        """Log-probs (+ entropy) of the response tokens, or values for the critic, from final hidden states."""
        h = self.ps.sp_gather(hidden)[pb.gather_index]
        if self.role == "critic":
            return self.model.value_head(h.float()).squeeze(-1), None
        temp = getattr(self.args, "rollout_temperature", 1.0)
        return self.ps.vocab_parallel_logprob(h, self.model.head_weight(), pb.targets, temp, with_entropy, self.cfg.vocab_size)

    def _forward_logprobs_cp(self, pb: PackedBatch, with_entropy: bool, replay: bool):
        """Context-parallel forward: this rank runs tokens [lo, hi) of the packed batch, scores the response tokens whose
        predicting row falls in that chunk, and the per-token results are assembled over the CP group (every rank ends
        with the full vectors, so sequence-level losses need no further communication)."""
        from ..parallel import cp, cp_ring

        ps = self.ps
        T = pb.tokens.numel()
        # the tokens this rank runs: a contiguous chunk (Ulysses, all-gather CP) or two zigzag pieces (ring CP)
        own = cp_ring.token_index(T, ps, pb.tokens.device)
        local_row = torch.full((T,), -1, dtype=torch.long, device=own.device)
        local_row[own] = torch.arange(own.numel(), device=own.device)
        rec = getattr(self.args, "recompute_granularity", None) == "full"
        meta = ForwardMeta(positions=pb.positions[own], cu_seqlens=pb.cu_seqlens, max_seqlen=pb.max_seqlen,
                           replay_topk=pb.replay_topk[own] if (replay and pb.replay_topk is not None) else None, recompute=rec)
        hidden = ps.sp_gather(self.model(pb.tokens[own], meta))
        rows = local_row[pb.gather_index]
        mine = rows >= 0
        h = hidden[rows[mine]]
        R = pb.gather_index.numel()
        if self.role == "critic":
            return cp.gather_from_cp(self.model.value_head(h.float()).squeeze(-1), mine, R, ps), None
        temp = getattr(self.args, "rollout_temperature", 1.0)
        lp, ent = ps.vocab_parallel_logprob(h, self.model.head_weight(), pb.targets[mine], temp, with_entropy, self.cfg.vocab_size)
        lp = cp.gather_from_cp(lp.float(), mine, R, ps)
        ent = cp.gather_from_cp(ent.float(), mine, R, ps) if ent is not None else None
        return lp, ent

    @torch.no_grad()
    def compute_log_probs(self, shard: dict, micro_batches: list[list[int]], tag: str | None = None) -> list[list[float]]:
        """Forward-only pass; returns per-sample log-prob lists aligned with the shard order."""
        if tag is not None and tag != "actor":
            self.backuper.backup("actor")
            self.backuper.restore(tag)
        out: dict[int, torch.Tensor] = {}
        replay = getattr(self.args, "use_routing_replay", False)
        self.model.eval()

        def pack(idx):
            return pack_micro_batch(shard, idx, self.device, pad_multiple=self._pad_multiple(), with_replay=replay)

        def keep(pb, idx, lp):
            for i, piece in zip(idx, lp.float().split(pb.response_lengths)):
                out[i] = piece

        batches = self.profiler.iterate("train_log_probs", micro_batches) if hasattr(self, "profiler") else micro_batches
        self._step_runner().forward_only_step(batches, pack, keep, replay=replay)
        if tag is not None and tag != "actor":
            self.backuper.restore("actor")
        return [out[i] for i in sorted(out)]

    def _pad_multiple(self) -> int:
        zigzag = 2 if (self.ps.cp_size > 1 and self.ps.cp_comm_type in ("p2p", "a2a+p2p")) else 1     # ring CP: two pieces per rank
        mult = int(getattr(self.args, "data_pad_size_multiplier", 128) or 128)
        return max(1, self.ps.tp_size) * max(1, self.ps.cp_size) * zigzag * (mult if self.device.type == "cuda" else 1)

    # ---------------------------------------------------------------------------------------
    # train
    # ---------------------------------------------------------------------------------------
    def train(self, rollout_id: int, shard: dict[str, Any]) -> dict[str, float]:
        """One rollout's worth of optimisation on this rank's data shard."""
        args = self.args
        if self.asleep:
            self.wake_up()
        t0 = time.time()
        n = len(shard["tokens"])
        dev = self.device
        ps = self.ps
        dp_group = ps.dp_group
        if ps.fabric is not None:
            ps.fabric.phase_barrier()       # absorb host skew between ranks before the first kernel that waits on a peer
        if getattr(self, "phase_sink", None) is not None:
            self.phase_sink.rollout_id = rollout_id
        with self.timer.span("data_preprocess"):
            mbs = make_micro_batches(args, shard["total_lengths"], dp_group=dp_group, cp_size=ps.cp_size)
        metrics: dict[str, float] = {}
        # ---- forward-only passes ----------------------------------------------------------
        ref_lp = old_lp = None
        if self.role == "actor":
            if getattr(args, "need_ref", False) and self.backuper.has("ref"):
                with self.timer.span("ref_log_probs"):
                    ref_lp = self.compute_log_probs(shard, mbs, tag="ref")
            if self.backuper.has("teacher") and "teacher_log_probs" not in shard:
                # --opd-type megatron: the teacher is a second set of weights of this trainer, scored like the reference policy
                with self.timer.span("teacher_log_probs"):
                    shard["teacher_log_probs"] = [t.tolist() for t in self.compute_log_probs(shard, mbs, tag="teacher")]
            if not getattr(args, "skip_actor_forward_only", False) and not getattr(args, "use_rollout_logprobs", False):
                self._hook("custom_megatron_before_log_prob_hook_path", rollout_id)
                with self.timer.span("log_probs"), self.profiler.range("log_probs"):
                    old_lp = self.compute_log_probs(shard, mbs, tag=None)
            elif getattr(args, "use_rollout_logprobs", False):
                assert "rollout_log_probs" in shard, "--use-rollout-logprobs needs engine log-probs"
        values = None
        if self.role == "critic" or "values" in shard:
            values = shard.get("values")
            if values is None:
                with self.timer.span("values"):
                    values = self.compute_log_probs(shard, mbs, tag=None)
                shard["values"] = values
        # ---- advantages ---------------------------------------------------------------------
        order = list(range(n))
        resp = shard["response_lengths"]
        lm_flat = flat_per_token(shard, "loss_masks", order, dev)
        if "advantages" not in shard:
            lp_flat = torch.cat(old_lp) if old_lp else (flat_per_token(shard, "rollout_log_probs", order, dev)
                                                        if "rollout_log_probs" in shard else None)
            ref_flat = torch.cat(ref_lp) if ref_lp else None
            val_flat = torch.cat([torch.as_tensor(v, device=dev, dtype=torch.float32) for v in values]) if values is not None else None
            adv, ret = compute_advantages_and_returns(
                args, rewards=torch.tensor(shard["rewards"], device=dev), response_lengths=resp, loss_mask=lm_flat,
                log_probs=lp_flat, ref_log_probs=ref_flat, values=val_flat, dp_group=dp_group,
                teacher_log_probs=flat_per_token(shard, "teacher_log_probs", order, dev) if "teacher_log_probs" in shard else None,
                opd_reverse_kl=flat_per_token(shard, "opd_reverse_kl", order, dev) if "opd_reverse_kl" in shard else None)
            shard["advantages"] = list(adv.split(resp))
            shard["returns"] = list(ret.split(resp))
        pattern = getattr(args, "save_debug_train_data", None)
        if pattern:
            path = pattern.format(rollout_id=rollout_id, rank=ps.rank)
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
            keep = ("tokens", "response_lengths", "total_lengths", "loss_masks", "rewards", "raw_reward", "rollout_log_probs", "sample_indices")
            blob = {k: shard[k] for k in keep if k in shard}
            blob["advantages"] = [a.tolist() for a in shard["advantages"]]
            blob["log_probs"] = [t.tolist() for t in old_lp] if old_lp else None
            blob["ref_log_probs"] = [t.tolist() for t in ref_lp] if ref_lp else None
            torch.save({"rollout_id": rollout_id, "rank": ps.rank, "dp_rank": ps.dp_rank, "data": blob}, path)
        if getattr(args, "ci_test", False) and old_lp is not None and ref_lp is not None and rollout_id == 0 \
                and not getattr(args, "ref_load", None):
            kl0 = (torch.cat(old_lp) - torch.cat(ref_lp)).abs().max().item()
            assert kl0 < 1e-5, f"KL between actor and reference must be 0 at step 0, got {kl0}"
        # ---- optimisation -------------------------------------------------------------------
        steps = max(1, getattr(args, "num_steps_per_rollout", 1) or 1)
        self.model.train()
        agg: dict[str, list] = {}
        with self.timer.span("actor_train" if self.role == "actor" else "critic_train"), self.profiler.range("actor_train"):
            per_step = _split_steps(mbs, steps)
            for step_mbs in self.profiler.iterate("train_actor", per_step):
                self._hook("custom_megatron_before_train_step_hook_path", rollout_id)
                step_metrics = self._train_one_step(shard, step_mbs, old_lp, ref_lp)
                for k, v in step_metrics.items():
                    agg.setdefault(k, []).append(v)
        for k, v in agg.items():
            metrics[f"train/{k}"] = float(sum(v) / len(v))
        metrics["perf/train_time"] = time.time() - t0
        tok = float(sum(shard["total_lengths"]))
        metrics["perf/actor_train_tok_per_s"] = tok / max(metrics["perf/train_time"], 1e-9)
        for k, v in self.timer.pop_all().items():
            metrics[f"perf/{k}_time"] = v
        if ps.fabric is not None:
            ps.fabric.check()               # a bounded wait on a peer ran out somewhere in this step: fail it loudly
        self.profiler.step(rollout_id)
        if "witness_ids" in shard and getattr(args, "audit_dir", None):
            from ..audit.events import DataWitness
            from ..orchestration.wiring import audit_logger

            DataWitness(audit_logger(args, "trainer", ps.rank)).consumed(rollout_id, self.global_step, shard["witness_ids"],
                                                                        dp_rank=ps.dp_rank)
        self.weight_version += 1
        return metrics

    def _train_one_step(self, shard, mbs: list[list[int]], old_lp, ref_lp) -> dict[str, float]:
        args, ps, dev = self.args, self.ps, self.device
        self.optimizer.zero_grad()
        replay = getattr(args, "use_routing_replay", False)
        # global batch of this optimizer step = Σ over DP ranks of local samples
        local_n = sum(len(m) for m in mbs)
        local_tok = sum(sum(shard["loss_masks"][i]) for m in mbs for i in m)
        counts = torch.tensor([float(local_n), float(local_tok)], device=dev)
        if ps.dp_size > 1 and ps.dp_group is not None:
            dist.all_reduce(counts, group=ps.dp_group)
        gbs, gtok = max(1.0, counts[0].item()), max(1.0, counts[1].item())
        sums: dict[str, torch.Tensor] = {}
        count_sum = torch.zeros((), device=dev)
        want_entropy = (getattr(args, "entropy_coef", 0.0) != 0 or getattr(args, "log_entropy", True)
                        or getattr(args, "observe_training_entropy", False))
        want_ent = want_entropy and self.role == "actor"

        def score(pb, idx, out, ent):
            """Loss of one micro-batch from its log-probs (values for the critic); adds its metrics to the step's sums."""
            nonlocal count_sum
            if not idx:                # empty micro-batch keeps collectives aligned across DP ranks
                return out.sum() * 0.0
            lb = LossBatch(
                response_lengths=pb.response_lengths, loss_mask=pb.loss_mask, seq_ids=pb.seq_ids,
                advantages=_cat(shard.get("advantages"), idx, dev), returns=_cat(shard.get("returns"), idx, dev),
                old_log_probs=_cat(old_lp, idx, dev) if old_lp is not None else None,
                ref_log_probs=_cat(ref_lp, idx, dev) if ref_lp is not None else None,
                rollout_log_probs=flat_per_token(shard, "rollout_log_probs", idx, dev),
                old_values=_cat(shard.get("values"), idx, dev) if self.role == "critic" else None,
                denominators=torch.tensor([shard["rollout_mask_sums"][i] for i in idx], device=dev, dtype=torch.float32)
                if "rollout_mask_sums" in shard else None)
            loss, m, count = loss_function(self._loss_args(), lb, out, ent, global_batch_size=gbs,
                                           global_num_tokens=gtok)
            aux = getattr(self.model, "aux_losses", None)
            if aux is not None and self.role == "actor":
                # model-side objectives of other families (the sparse-attention indexer's KL), weighted like one micro-batch
                for name, term in aux().items():
                    loss = loss + getattr(args, "aux_loss_coef", 1.0) * term / max(1, len(mbs))
                    m[name] = term.detach() * count
            for k, v in m.items():
                sums[k] = sums.get(k, 0) + v.detach().float()
            count_sum = count_sum + count
            return loss

        def pack(idx):
            return pack_micro_batch(shard, idx, dev, pad_multiple=self._pad_multiple(), with_replay=replay)

        # the schedule of forwards and backwards over the micro-batches belongs to the step runner (linear, GPipe, 1F1B, or
        # a custom one): this method only says how a micro-batch is packed and how its loss is computed
        runner = self._step_runner()
        runner.forward_backward_step(mbs, pack, score, want_ent=want_ent, replay=replay)
        self._finalize_grads()
        if self.dumper is not None:
            with self.dumper.phase("fwd_bwd") as d:
                if d is not None:
                    d.dump_model(self.model)                 # parameters and the reduced gradients of this optimizer step
                    d.step()
        lr = self.scheduler.get()
        if getattr(args, "debug_disable_optimizer", False):
            self.optimizer.zero_grad()
            stats = {"grad_norm": 0.0}
        elif self._exchange_across_cells():
            stats = self.optimizer.step(lr)
            self.scheduler.step()
            self.global_step += 1
        else:
            # the cells agreed to discard this step (some cell saw a non-finite gradient): nothing is applied anywhere
            self.optimizer.zero_grad()
            stats = {"grad_norm": float("nan")}
        # metrics: Σ over micro-batches and DP ranks of reduced values / global count
        keys = sorted(sums)
        if ps.dp_size > 1 and ps.dp_group is not None:
            # ranks may have seen different key sets only if some had empty batches; unify by name
            all_keys = [None] * ps.dp_size
            dist.all_gather_object(all_keys, keys, group=ps.dp_group)
            keys = sorted(set(k for ks in all_keys for k in ks))
        vec = torch.stack([count_sum] + [torch.as_tensor(sums.get(k, 0.0), device=dev, dtype=torch.float32) for k in keys]) \
            if keys else count_sum[None]
        if ps.dp_size > 1 and ps.dp_group is not None:
            dist.all_reduce(vec, group=ps.dp_group)
        denom = vec[0].clamp_min(1.0)
        out_metrics = {k: (vec[1 + j] / denom).item() for j, k in enumerate(keys)}
        if ps.pp_size > 1:                        # losses exist on the last stage only
            box = [out_metrics]
            dist.broadcast_object_list(box, src=ps.pp_ranks[-1], group=ps.pp_group)
            out_metrics = box[0]
        out_metrics["grad_norm"] = stats["grad_norm"]
        out_metrics["lr-pg_0"] = lr
        return out_metrics

    def _step_runner(self):
        """The object that runs forwards and backwards over micro-batches (`train/step_runner.py`); `--custom-step-runner-path`
        plugs another schedule or another backend's model."""
        r = getattr(self, "_runner", None)
        if r is None:
            from .step_runner import build_step_runner

            r = self._runner = build_step_runner(self)
        return r

    def _loss_args(self):
        if self.role != "critic":
            return self.args
        a = Namespace(**vars(self.args))
        a.loss_type = "value_loss"
        return a

    def _finalize_grads(self):
        """Sum the partial gradients of tensor-parallel-replicated parameters over the TP group
        (each TP rank saw a different sequence slice under sequence parallelism)."""
        ps = self.ps
        if ps.tp_size > 1 and ps.tp_group is not None:
            grads = [p.main_grad for n, p in self.model.named_parameters() if n in self.tp_replicated and p.requires_grad]
            if grads:
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=ps.tp_group)
                off = 0
                for g in grads:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()

    # ---------------------------------------------------------------------------------------
    # weights: export / sync / save / sleep
    # ---------------------------------------------------------------------------------------
    def update_weights(self, engine_or_updater) -> dict:
        """Push current weights to the rollout engine(s); see `miles_b200.weight_update`."""
        from ..weight_update.updater import WeightUpdater

        upd = engine_or_updater if isinstance(engine_or_updater, WeightUpdater) else \
            WeightUpdater(self.args, self, engine_or_updater)
        temporary = getattr(self, "_groups_released", False)     # asleep with released groups: bring them back for the transfer
        self.ensure_groups()
        with self.timer.span("update_weights"):
            if getattr(self.model, "lora_adapters", None) and upd.mode != "alias":
                from .lora import merged
                with merged(self.model):          # the engine serves base + adapter as one set of weights
                    info = upd.update_weights()
            else:
                info = upd.update_weights()
        if temporary:
            self._groups_released = self.ps.release_groups() > 0
        return info

    def save_model(self, iteration: int, with_optimizer: bool = True):
        from ..checkpoint import manager as ckpt
        self.ensure_groups()
        ckpt.save_from_actor(self, self.args, iteration, with_optimizer)
        if getattr(self.args, "save_local_weight_checksum", False):
            from ..audit.events import combined_checksum, model_checksums
            import json
            import os

            sums = model_checksums(self.named_weights())
            d = ckpt.iter_dir(self.args.save, iteration)
            with open(os.path.join(d, f"weight_checksum_rank{self.ps.rank:05d}.json"), "w") as f:
                json.dump({"combined": combined_checksum(sums), "tensors": sums}, f)
        self._hook("custom_megatron_post_save_hook_path", iteration)

    def sleep(self, tags=("optimizer", "grad")):
        """Release trainer memory for the rollout phase (colocated mode): optimizer shards move to
        pinned host memory, gradient buffers are dropped; the bf16 weights stay (the engine reads them)."""
        from ..utils.memory import offload_tensors
        if self.asleep:
            return
        groups = self.optimizer.tensors_by_tag()
        self._offloaded = {}
        if "optimizer" in tags:
            if getattr(self, "arena", None) is not None:
                self._arena_released = self.arena.pause("optimizer", keep_contents=True)
            else:
                self._offloaded["optimizer"] = offload_tensors(groups["optimizer"])
        if "grad" in tags:
            self.optimizer.release_grads()
        if getattr(self.args, "offload_train_release_process_groups", False):
            # communicators pin device memory too; with engines in other processes nothing here needs them until wake-up
            self._groups_released = self.ps.release_groups() > 0
        self.asleep = True

    def wake_up(self):
        from ..utils.memory import onload_tensors
        if not self.asleep:
            self.ensure_groups()
            return
        self.ensure_groups()
        if getattr(self, "arena", None) is not None and getattr(self, "_arena_released", 0):
            self.arena.resume("optimizer")
            self._arena_released = 0
        for t, saved in self._offloaded.items():
            onload_tensors(saved)
        self._offloaded = {}
        self.optimizer.restore_grads()
        self.asleep = False

    def _nvme_dir(self):
        """`--optimizer-nvme-dir DIR` (or `--stream-optimizer-state-to-disk`, which defaults DIR to <save>/optimizer_stream)."""
        d = getattr(self.args, "optimizer_nvme_dir", None)
        if d is None and getattr(self.args, "stream_optimizer_state_to_disk", False):
            import tempfile

            base = getattr(self.args, "save", None) or tempfile.gettempdir()
            d = os.path.join(base, "optimizer_stream")
        return os.path.join(d, self.role) if d else None

    def ensure_groups(self):
        """Re-create the process groups released by `sleep` (collective; a no-op when they are alive)."""
        if getattr(self, "_groups_released", False):
            self.ps.reload_groups()
            self._groups_released = False

    def named_weights(self):
        """This rank's shard, named by our layout (for checkpointing and weight sync).  With the FSDP backend every
        parameter is gathered in full, one at a time (collective: all ranks iterate together)."""
        if getattr(self, "fsdp", False):
            from .fsdp import full_data

            return ((n, full_data(p)) for n, p in self.model.named_parameters_global())
        return [(n, p.data) for n, p in self.model.named_parameters_global()]


def _tp_replicated(name: str) -> bool:
    last = name.rsplit(".", 1)[-1]
    if ".value_head." in name or (".lora." in name and last.endswith("_r")):
        return True
    return last in ("ln1", "ln2", "norm", "q_norm", "k_norm", "router")


def _cat(lst, idx, dev):
    if lst is None:
        return None
    parts = [torch.as_tensor(lst[i], device=dev, dtype=torch.float32) for i in idx]
    return torch.cat(parts) if parts else torch.zeros(0, device=dev)


def _split_steps(mbs: list[list[int]], steps: int) -> list[list[list[int]]]:
    """Distribute micro-batches over `steps` optimizer steps (contiguous, as even as possible)."""
    if steps <= 1:
        return [mbs]
    flat = [i for m in mbs for i in m]
    per = (len(flat) + steps - 1) // steps
    mb_size = max(1, max((len(m) for m in mbs), default=1))
    out = []
    for s in range(steps):
        chunk = flat[s * per:(s + 1) * per]
        out.append([chunk[i:i + mb_size] for i in range(0, len(chunk), mb_size)] or [[]])
    return out
