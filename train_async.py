"""Asynchronous RL training loop: rollout N+1 is generated while the trainer works on rollout N.

Same contract as the reference's `train_async.py` (train_async.py:23-132): `--colocate` is rejected (the engine must
keep serving while the trainer computes, so it owns its weights and KV memory); by default the in-flight rollout is
drained before a weight update so that every sample of a batch comes from one weight version; with `--fully-async`
generation continues across updates (a persistent producer with a staleness-bounded buffer,
`miles_b200.rollout.fully_async`) and samples record the versions they span.

The engine runs on a thread of this process with its own CUDA stream of work (or behind `--rollout-engine http`);
torchrun launches one such process per GPU as for `train.py`.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

from miles_b200.args import parse_args
from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_training_models,
                                             update_weights)
from miles_b200.utils import object_store
from miles_b200.utils.tracking import Tracker


def _should(interval, i, total=None):
    if not interval:
        return False
    return (i + 1) % interval == 0 or (total is not None and i + 1 == total)


def train(args):
    assert not args.colocate, "train_async.py needs the engine to keep its own memory: drop --colocate"
    ps = create_parallel_state(args)
    assert getattr(args, "rollout_engine", "native") == "http" or (ps.tp_size == 1 and ps.ep_size == 1), \
        "the in-process engine thread may not issue collectives concurrently with the trainer; use --rollout-engine http"
    tracker = Tracker(args, stdout=ps.rank == 0)
    args.engine_kwargs = dict(getattr(args, "engine_kwargs", {}) or {}, own_weights=True)
    if args.fully_async and getattr(args, "rollout_function_path", None) in (
            None, "miles_b200.rollout.inference_rollout.InferenceRolloutFn"):
        args.rollout_function_path = "miles_b200.rollout.fully_async.FullyAsyncRolloutFn"
    actor, critic, start = create_training_models(args, ps)
    rollout = create_rollout_components(args, ps, actor, tracker)
    rollout.executor.load(start - 1 if start > 0 else None)
    if args.num_rollout is None:
        assert args.num_epoch and len(rollout.data_source), "--num-rollout or --num-epoch (with --prompt-data) required"
        args.num_rollout = args.num_epoch * len(rollout.data_source) // args.rollout_batch_size
    update_weights(args, actor, rollout)

    pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="rollout")
    try:
        nxt = pool.submit(rollout.executor.get, start) if start < args.num_rollout else None
        for rollout_id in range(start, args.num_rollout):
            pack = nxt.result()
            # generation of the next batch overlaps everything below
            nxt = pool.submit(rollout.executor.get, rollout_id + 1) if rollout_id + 1 < args.num_rollout else None
            shard = object_store.get(pack.data_ref)
            metrics = dict(pack.metrics)
            if critic is not None:
                cm = critic.train(rollout_id, shard)
                metrics.update({k.replace("train/", "train/critic-"): v for k, v in cm.items()})
            if critic is None or rollout_id >= args.num_critic_only_steps:
                metrics.update(actor.train(rollout_id, shard))
            object_store.remove(pack.data_ref)
            if args.save and _should(args.save_interval, rollout_id, args.num_rollout):
                actor.save_model(rollout_id)
                rollout.executor.save(rollout_id)
            if _should(args.update_weights_interval, rollout_id):
                if not args.fully_async and nxt is not None:
                    nxt.result()              # drain: the batch in flight finishes on the old weights
                info = update_weights(args, actor, rollout)
                metrics["perf/update_weights_time"] = info["seconds"]
            if _should(args.eval_interval, rollout_id) and not args.fully_async:
                if nxt is not None:
                    nxt.result()
                metrics.update(rollout.executor.eval(rollout_id))
            tracker.log(metrics, rollout_id)
    finally:
        rollout.executor.shutdown()
        pool.shutdown(wait=True)
    from miles_b200.checkpoint.manager import finalize_async_save

    finalize_async_save()                 # --async-save: the last checkpoint is on disk before the run ends
    if getattr(rollout, "fleet", None) is not None:
        rollout.fleet.shutdown()          # engine servers and router launched by this job
    tracker.finish()
    return tracker


if __name__ == "__main__":
    os.environ.setdefault("MILES_ASYNC", "1")
    train(parse_args())
