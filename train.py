"""Synchronous (optionally colocated) RL training loop.

    rollout → [offload rollout / onload train] → critic/actor train → save → [offload train / onload
    rollout] → update_weights → eval

Same loop and flags as the reference's `train.py` (train.py:25-176); launch one process per GPU with
torchrun (`python -m torch.distributed.run --nproc-per-node N train.py …`) or run directly on one
device / CPU.
"""
from __future__ import annotations

import os

from miles_b200.args import parse_args
from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_trainer_controller,
                                             create_training_models, update_weights)
from miles_b200.utils import object_store
from miles_b200.utils.tracking import Tracker


def _should(interval, i, total=None):
    if not interval:
        return False
    return (i + 1) % interval == 0 or (total is not None and i + 1 == total)


def train(args):
    ps = create_parallel_state(args)
    tracker = Tracker(args, stdout=ps.rank == 0)
    actor, critic, start_rollout_id = create_training_models(args, ps)
    trainer = create_trainer_controller(args, actor)     # retries / heartbeats under --use-fault-tolerance, else a pass-through
    rollout = create_rollout_components(args, ps, actor, tracker)
    rollout.executor.load(start_rollout_id - 1 if start_rollout_id > 0 else None)
    if args.num_rollout is None:
        assert args.num_epoch and len(rollout.data_source), "--num-rollout or --num-epoch (with --prompt-data) required"
        args.num_rollout = args.num_epoch * len(rollout.data_source) // args.rollout_batch_size

    from miles_b200.ft.api_server import maybe_start_mini_ft_controller, start_api_server

    api = start_api_server(args, trainer, rollout) if ps.rank == 0 else None     # --api-server-port: cells over REST
    maybe_start_mini_ft_controller(args) if api else None
    if not args.debug_train_only and not args.debug_skip_weight_update:
        update_weights(args, actor, rollout)           # initial push (and consistency check)
    if args.offload_train and not args.debug_rollout_only:
        actor.sleep()
    if args.eval_interval and not args.skip_eval_before_train and start_rollout_id == 0:
        rollout.executor.eval(0)

    for rollout_id in range(start_rollout_id, args.num_rollout):
        pack = rollout.executor.get(rollout_id)
        if args.debug_rollout_only:
            tracker.log(pack.metrics, rollout_id)
            continue
        if args.colocate and args.offload_rollout:
            rollout.controller.offload(("kv_cache", "cuda_graph"))
        shard = object_store.get(pack.data_ref)
        metrics = dict(pack.metrics)
        if critic is not None:
            cm = critic.train(rollout_id, shard)
            metrics.update({k.replace("train/", "train/critic-"): v for k, v in cm.items()})
        if critic is None or rollout_id >= args.num_critic_only_steps:
            metrics.update(trainer.train(rollout_id, shard))
        object_store.remove(pack.data_ref)

        sentinel = args.save_trigger_sentinel and os.path.exists(args.save_trigger_sentinel)
        if args.save and (_should(args.save_interval, rollout_id, args.num_rollout) or sentinel):
            actor.save_model(rollout_id)
            rollout.executor.save(rollout_id)
            if sentinel and ps.rank == 0:
                os.remove(args.save_trigger_sentinel)

        if args.offload_train:
            actor.sleep()
        if _should(args.update_weights_interval, rollout_id) and not args.debug_skip_weight_update:
            info = update_weights(args, actor, rollout)
            metrics["perf/update_weights_time"] = info["seconds"]
        if args.colocate and args.offload_rollout:
            rollout.controller.onload(("weights", "kv_cache", "cuda_graph"))
        if _should(args.eval_interval, rollout_id):
            metrics.update(rollout.executor.eval(rollout_id))
        tracker.log(metrics, rollout_id)
        if args.debug_exit_after_rollout is not None and rollout_id >= args.debug_exit_after_rollout:
            break
    if args.enable_event_analyzer and args.audit_dir and ps.rank == 0:
        from miles_b200.audit import events

        findings = events.analyze(args.audit_dir)
        tracker.findings = findings
        if findings:
            print(f"[audit] {len(findings)} finding(s): " + "; ".join(str(dict(f)) for f in findings[:5]))
    from miles_b200.checkpoint.manager import finalize_async_save

    finalize_async_save()                 # --async-save: the last checkpoint is on disk before the run ends
    if getattr(rollout, "fleet", None) is not None:
        rollout.fleet.shutdown()          # engine servers and router launched by this job
    tracker.finish()
    tracker.actor = actor          # programmatic callers (tests, notebooks) reach the trained model through the tracker
    return tracker


if __name__ == "__main__":
    train(parse_args())
