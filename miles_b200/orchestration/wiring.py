"""Wiring helpers used by the entry points: parallel state, trainer(s), rollout components, weight push.

Names follow the reference's helpers (`create_rollout_components`, `create_training_models`,
`update_weights`: miles/ray/placement_group.py:216-255,295-321,371-404).  Instead of Ray placement groups
the process model is SPMD — one process per GPU started by torchrun (or a single process on CPU) — and
the "controllers" are plain objects in each rank.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from ..args import model_config_from_args
from ..parallel.state import ParallelState, init_distributed


@dataclass
class RolloutComponents:
    engines: list
    client: Any
    executor: Any
    data_source: Any
    controller: Any = None          # InferenceController over `engines`: memory hand-over, weight-update framing, health
    fleet: Any = None               # workers.fleet.Fleet when engine servers run as supervised processes (HTTP engines)


def create_parallel_state(args) -> ParallelState:
    rank, world, local = init_distributed(backend=getattr(args, "distributed_backend", None),
                                          timeout_s=60.0 * (getattr(args, "distributed_timeout_minutes", 30) or 30))
    if world == 1:
        return ParallelState.single()
    ps = ParallelState.build(
        tp=args.tensor_model_parallel_size, cp=args.context_parallel_size, pp=args.pipeline_model_parallel_size,
        ep=args.expert_model_parallel_size, sequence_parallel=args.sequence_parallel, cp_comm_type=args.cp_comm_type,
        vpp=getattr(args, "virtual_pipeline_model_parallel_size", None) or 1,
        cp_hierarchy=tuple(args.hierarchical_context_parallel_sizes) if getattr(args, "hierarchical_context_parallel_sizes", None) else None)
    ps.fused = not getattr(args, "disable_fused_comm", False)
    if torch.cuda.is_available() and ps.fused and (ps.tp_size > 1 or ps.ep_size > 1 or ps.dp_size > 1):
        from ..parallel.fabric import Fabric

        ps.fabric = Fabric.create(ps)
    return ps


def apply_serving_config(args) -> None:
    """`--engine-config`: the server groups of the policy model (the first model that is not eval-only) decide how many
    engine servers the fleet starts and in which roles — `regular` engines behind the router (over `num_gpus_per_engine` GPUs each), or
    single-GPU `prefill` + `decode` engines with the KV hand-over between them."""
    from .inference_controller import load_serving_config

    models = load_serving_config(args.engine_config)
    policy = next((m for m in models if not m.eval_only), None)
    assert policy is not None, "--engine-config names no model that serves the policy"
    count = {"regular": 0, "prefill": 0, "decode": 0}
    per = {grp.num_gpus_per_engine for grp in policy.groups if grp.worker_type in count}
    assert len(per) <= 1, f"{policy.name}: the groups of one fleet use one engine size, got {sorted(per)}"
    if per:
        args.rollout_num_gpus_per_engine = per.pop()
        assert args.rollout_num_gpus_per_engine == 1 or not any(g.worker_type == "prefill" for g in policy.groups), \
            "prefill / decode roles run on single-GPU engine servers"
    for grp in policy.groups:
        if grp.worker_type in count:
            count[grp.worker_type] += grp.num_gpus // grp.num_gpus_per_engine
    if count["prefill"]:
        assert not count["regular"], f"{policy.name}: regular groups next to prefill / decode groups are not supported"
        args.rollout_num_engines = count["prefill"] + count["decode"]
        args.rollout_pd_prefill_engines = count["prefill"]
    elif count["regular"]:
        args.rollout_num_engines = count["regular"]
    if policy.model_path and not getattr(args, "hf_checkpoint", None):
        args.hf_checkpoint = policy.model_path


def load_tokenizer(args):
    path = getattr(args, "tokenizer_path", None) or getattr(args, "hf_checkpoint", None)
    if not path or not os.path.isdir(path):
        return None
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(path, trust_remote_code=True)
    except Exception:
        return None


def create_training_models(args, ps: ParallelState):
    from ..train.actor import TrainActor

    actor = TrainActor(args, ps, role="actor")
    start = actor.init()
    critic = None
    if args.advantage_estimator == "ppo":
        critic = TrainActor(args, ps, role="critic")
        critic.init()
    return actor, critic, start


class TrainerController:
    """Driver-side handle of the trainer (reference: `TrainerController`, miles/ray/train/group.py:52-685).  Without
    `--use-fault-tolerance` calls go straight to this rank's `TrainActor`.  With it the actor is a `Cell` of a
    `CellController`: a call that raises is retried (`--ft-max-attempts`, the reference retries 30 times) after the
    cell's state was rolled back by `recover`, the membership epoch is published, and every step leaves a heartbeat in
    the job's store when one is configured (`--indep-dp-store`), which is what the health checker of the other cells and of
    an external supervisor read."""

    def __init__(self, args, actor):
        self.args, self.actor = args, actor
        self.cells = None
        self.monitor = None
        if getattr(args, "use_fault_tolerance", False):
            from ..ft.controller import Cell, CellController, HeartbeatMonitor

            cell_id = getattr(args, "indep_dp_cell_id", 0) or 0
            self.cells = CellController([Cell(cell_id, [_RetryableActor(actor)])], min_quorum=1,
                                        max_attempts=getattr(args, "ft_max_attempts", 30) or 30)
            store = getattr(actor, "cell_store", None)
            if store is not None:
                self.monitor = HeartbeatMonitor(store, timeout_s=getattr(args, "ft_heartbeat_timeout", 60.0) or 60.0)
            self.worker_id = f"cell{cell_id}/rank{actor.ps.rank}"

    def train(self, rollout_id: int, shard: dict) -> dict:
        if self.cells is None:
            return self.actor.train(rollout_id, shard)
        if self.monitor is not None:
            self.monitor.beat(self.worker_id)
        # one local cell: a failed attempt fences it (min_quorum = 1 makes `execute` give up at once); the worker is this very
        # process, still alive after a host-side exception, so it is re-admitted (`heal`) and the step is tried again
        last = None
        for _ in range(self.cells.max_attempts):
            try:
                out = self.cells.execute("train", rollout_id, shard)
                return next(iter(out.values()))[0]
            except RuntimeError as e:
                last = e
                dead = [c for c in self.cells.cells.values() if c not in self.cells.alive()]
                if not dead:
                    raise
                for c in dead:
                    self.cells.heal(c.cell_id, [_RetryableActor(self.actor)])
        raise RuntimeError(f"train did not succeed in {self.cells.max_attempts} attempts") from last

    def __getattr__(self, name):
        return getattr(self.actor, name)


class _RetryableActor:
    """A worker handle whose failed call leaves the trainer where it was: gradients cleared, nothing half applied."""

    def __init__(self, actor):
        self.actor = actor

    def init(self, *a, **kw):
        return None            # the actor of this process is initialised by `create_training_models`

    def train(self, rollout_id, shard):
        from ..testing import fault_injector

        try:
            fault_injector.GLOBAL.at("train", step=rollout_id)    # host-side injection point, before anything is launched
            return self.actor.train(rollout_id, shard)
        except BaseException:
            self.actor.optimizer.zero_grad()
            shard.pop("advantages", None)
            shard.pop("returns", None)
            raise

    def kill(self):
        return None            # fencing a cell of ONE process means not calling it again; the controller does that


def create_trainer_controller(args, actor) -> TrainerController:
    return TrainerController(args, actor)


def create_rollout_components(args, ps: ParallelState, actor=None, tracker=None) -> RolloutComponents:
    from ..engine.engine import Engine
    from ..rollout.client import HttpEngineClient, InProcEngineClient
    from ..utils.misc import load_function
    from .rollout_executor import RolloutExecutor

    cfg = actor.cfg if actor is not None else model_config_from_args(args)
    tok = load_tokenizer(args)
    ds_cls = load_function(args.data_source_path)
    data_source = ds_cls(args, tok)
    kind = getattr(args, "rollout_engine", "native")
    engines: list = []
    fleet = None
    if kind == "http":
        router_url = (getattr(args, "engine_kwargs", None) or {}).get("router_url")
        worker_urls = None
        if getattr(args, "engine_config", None):
            apply_serving_config(args)
        if getattr(args, "worker_provider", "none") != "none":
            # engine servers + router as supervised worker processes (or adopted from elsewhere): rank 0 owns the fleet,
            # the other ranks only learn the router's address
            from .workers.fleet import launch_fleet

            if ps.rank == 0:
                fleet = launch_fleet(args, log_dir=getattr(args, "worker_log_dir", None))
                engines = list(fleet.engines.values())
                router_url, worker_urls = fleet.router_url, [e.url for e in engines]
            if ps.world_size > 1:
                box = [router_url, worker_urls]
                torch.distributed.broadcast_object_list(box, src=0)
                router_url, worker_urls = box
        n_moe = sum(cfg.layer_is_moe(l) for l in range(cfg.num_layers))
        n_prefill = int(getattr(args, "rollout_pd_prefill_engines", 0) or 0)
        if n_prefill > 0:
            # prefill / decode disaggregation: the first engines of the fleet run prompts, the others continue from their KV
            from ..engine.pd import PDHttpClient

            assert worker_urls and 0 < n_prefill < len(worker_urls), "--rollout-pd-prefill-engines needs a fleet with more engines than that"
            client = PDHttpClient(worker_urls[:n_prefill], worker_urls[n_prefill:], tokenizer=tok, num_moe_layers=n_moe, moe_topk=cfg.moe_topk)
        else:
            client = HttpEngineClient(router_url, tokenizer=tok, worker_urls=worker_urls, num_moe_layers=n_moe, moe_topk=cfg.moe_topk)
    else:
        ek = dict(getattr(args, "engine_kwargs", {}) or {})
        device = actor.device if actor is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        dtype = (getattr(actor, "compute_dtype", None) or next(actor.model.parameters()).dtype) if actor is not None else torch.bfloat16
        share = actor is not None and getattr(args, "colocate", False) and not ek.get("own_weights", False)
        eos = ek.get("eos_token_ids") or ([tok.eos_token_id] if tok is not None and tok.eos_token_id is not None else [])
        engine_ps = ps
        if getattr(actor, "fsdp", False):
            # FSDP keeps parameters sharded between uses: the engine holds a copy of its own, fed by the named tensor stream
            share = False
        if ps.pp_size > 1:
            # a pipeline stage holds a slice of the layers: the in-process engine then keeps a full copy of its own
            # (every rank serves requests data-parallel) and receives weights through the HF-named tensor stream
            assert ps.tp_size == 1 and ps.ep_size == 1, "in-process engine under PP needs tp = ep = 1; use --rollout-engine http"
            engine_ps, share = ParallelState.single(), False
        engine = Engine(cfg, model=actor.model if share else None, ps=engine_ps, device=device, dtype=dtype,
                        num_blocks=ek.get("num_blocks"), block_size=ek.get("block_size"),
                        mem_fraction_static=ek.get("mem_fraction_static", 0.7),
                        max_running_requests=ek.get("max_running_requests", 512),
                        max_prefill_tokens=ek.get("max_prefill_tokens", 16384),
                        max_context_len=getattr(args, "rollout_max_context_len", None), eos_token_ids=eos, tokenizer=tok,
                        seed=args.rollout_seed, use_cuda_graph=not ek.get("disable_cuda_graph", False),
                        prefix_cache=not ek.get("disable_radix_cache", False),
                        chunked_prefill_size=(ek.get("chunked_prefill_size") if (ek.get("chunked_prefill_size") or 0) > 0 else None))
        engine.attach_dumper(getattr(actor, "dumper", None))
        engines = [engine]
        client = InProcEngineClient(engines, tokenizer=tok, policy=getattr(args, "router_policy", "least_active"))
    # rollout data parallelism: one engine group per (tp × ep-within-dp) block; groups take disjoint prompts
    # (ranks of one TP group replicate the same requests; EP is orthogonal: DP attention + EP experts)
    # (pipeline stages each own an engine, so they count as rollout-DP ranks too)
    rollout_dp = max(1, ps.world_size // ps.tp_size)
    rollout_dp_rank = ps.rank // ps.tp_size
    ex = RolloutExecutor(args, data_source, client, ps=ps, rollout_dp_size=rollout_dp, rollout_dp_rank=rollout_dp_rank,
                         tracker=tracker)
    ex.is_leader = ps.tp_rank == 0
    # distinct prompts per rollout-DP rank (and per independent-DP cell): advance the data source by rank-dependent seeds
    if hasattr(data_source, "gen"):
        cell = getattr(args, "indep_dp_cell_id", 0)
        data_source.gen.manual_seed(args.rollout_seed * 9973 + rollout_dp_rank + 7919 * cell)
    controller = None
    if engines:
        from .inference_controller import InferenceController, ServerCell, ServerGroup

        group = ServerGroup("regular", max(1, ps.tp_size), max(1, ps.tp_size))
        controller = InferenceController([ServerCell(e, "default", group) for e in engines],
                                         probe=lambda e: e.health().get("status") == "ok",
                                         health_threshold=getattr(args, "miles_router_health_check_failure_threshold", 3) or 3)
        controller.pause_mode = getattr(args, "pause_generation_mode", None) or "retract"
        if fleet is not None:
            # a cell restarted by the fleet watcher comes back with fresh weights: stale until the updater has re-sent them
            fleet.on_restart = lambda e: setattr(controller._cell_of(e), "state", "stale")
    return RolloutComponents(engines=engines, client=client, executor=ex, data_source=data_source, controller=controller,
                             fleet=fleet)


def update_weights(args, actor, rollout: RolloutComponents, updater=None) -> dict:
    """start_update_weights (pause + flush under the controller's lock) → actor.update_weights → end_update_weights
    (version label + resume; engines resume on their old version when the transfer failed), then the new weight version is
    published to the executor (reference: miles/ray/placement_group.py:371-404)."""
    from ..weight_update.updater import WeightUpdater

    updater = updater or WeightUpdater(args, actor, rollout.engines)
    ctl = getattr(rollout, "controller", None)
    if ctl is None:
        info = actor.update_weights(updater)
    else:
        ctl.tick()                                         # quarantine engines that stopped answering before talking to them
        targets = ctl.start_update_weights()
        ok = False
        try:
            updater.framed = True                          # the controller owns pause / flush / resume for this transfer
            updater.engines = list(targets) or updater.engines
            info = actor.update_weights(updater)
            ok = True
        finally:
            updater.framed = False
            ctl.end_update_weights(actor.weight_version, ok=ok)
        for e in ctl.stale_engines():                      # re-admitted engines that missed updates are now in line
            ctl.mark_synced(e)
    rollout.executor.set_weight_version(actor.weight_version)
    if getattr(args, "audit_dir", None):
        _audit_weights(args, actor, rollout, info)
    if getattr(args, "snapshot_dir", None):
        info["snapshot"] = _publish_snapshot(args, actor)
    return info


_SNAPSHOTS = {}


def _publish_snapshot(args, actor):
    """Periodic full HF export next to the weight push (engines outside the job follow `latest`); every trainer rank drives
    the HF-named bucket iterator (its shard gathers are collective), rank 0 writes."""
    from ..weight_update.delta import SnapshotPublisher
    from ..weight_update.hf_iterator import iter_hf_weights

    pub = _SNAPSHOTS.get(args.snapshot_dir)
    if pub is None:
        pub = _SNAPSHOTS[args.snapshot_dir] = SnapshotPublisher(args.snapshot_dir, actor.cfg, every=args.snapshot_interval,
                                                                keep=args.snapshot_keep, src_dir=getattr(args, "hf_checkpoint", None))
    rank0 = not dist.is_initialized() or dist.get_rank() == 0
    return pub.maybe_publish(actor.weight_version, iter_hf_weights(actor, bucket_bytes=getattr(args, "update_weight_buffer_size", 512 << 20)),
                             write=rank0)


_AUDIT = {}


def audit_logger(args, source: str, rank: int):
    """One JSONL event log per (source, rank) under `--audit-dir` (see `miles_b200.audit.events`)."""
    from ..audit.events import EventLogger

    key = (args.audit_dir, source, rank)
    if key not in _AUDIT:
        _AUDIT[key] = EventLogger(args.audit_dir, source, rank)
    return _AUDIT[key]


def _audit_weights(args, actor, rollout: RolloutComponents, info: dict):
    """Checksums of what the trainer published and of what each in-process engine now holds (same layout only)."""
    from ..audit.events import combined_checksum, model_checksums

    rank = actor.ps.rank
    mine = combined_checksum(model_checksums(actor.named_weights()))
    audit_logger(args, "trainer", rank).log("weights_published", version=actor.weight_version, checksum=mine, mode=info.get("mode"))
    for i, e in enumerate(rollout.engines):
        model = getattr(e, "model", None)
        if model is None or info.get("mode") not in ("alias", "nvlink"):
            continue
        named = model.named_parameters_global() if hasattr(model, "named_parameters_global") else model.named_parameters()
        got = combined_checksum(model_checksums((n, p.data) for n, p in named if ".lora." not in n or info.get("mode") == "alias"))
        audit_logger(args, "engine", rank).log("weights_received", version=actor.weight_version, checksum=got, engine=f"rank{rank}#{i}")
