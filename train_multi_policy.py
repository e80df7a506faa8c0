"""Train several policies concurrently, one asyncio task per policy, with leader/follower barriers for save and eval.

Counterpart of the reference's `train_multi_policy.py` (train_multi_policy.py:32-213, miles/utils/multi_policy/*): each
policy has its own trainer, rollout components, data source and checkpoint directory; all of them advance in lock-step
per rollout id where the job needs a common point (saving a consistent set of checkpoints, evaluating policies against
each other), which the `Parker` provides: every policy parks at the barrier, the leader runs the critical section once,
then all resume.

    python train_multi_policy.py --multi-policy-config policies.yaml <common flags>

`policies.yaml`: a list of `{name: …, overrides: {flag_name: value, …}}`; every policy starts from the common flags.
Policies share the process (and GPU): their models live side by side, their steps interleave at `await` points.
"""
from __future__ import annotations

import asyncio
import copy
import os

import yaml

from miles_b200.args import build_parser, parse_args, validate_args
from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_training_models,
                                             update_weights)
from miles_b200.utils import object_store
from miles_b200.utils.tracking import Tracker


class Parker:
    """Reusable barrier for `n` asyncio tasks: the last arrival runs `leader_fn` (if given), then everyone resumes."""

    def __init__(self, n: int):
        self.n = n
        self._count = 0
        self._gen = 0
        self._cond = asyncio.Condition()
        self.passes = 0

    async def park(self, leader_fn=None):
        async with self._cond:
            gen = self._gen
            self._count += 1
            if self._count == self.n:
                if leader_fn is not None:
                    r = leader_fn()
                    if asyncio.iscoroutine(r):
                        await r
                self._count = 0
                self._gen += 1
                self.passes += 1
                self._cond.notify_all()
            else:
                await self._cond.wait_for(lambda: self._gen != gen)

    def leave(self):
        """A policy that finished early stops taking part."""
        self.n -= 1


def load_policy_args(common, path: str) -> list:
    with open(path) as f:
        spec = yaml.safe_load(f)
    out = []
    for i, p in enumerate(spec):
        a = copy.deepcopy(common)
        a.policy_name = p.get("name", f"policy{i}")
        for k, v in (p.get("overrides") or {}).items():
            setattr(a, k.replace("-", "_"), v)
        if a.save:
            a.save = os.path.join(a.save, a.policy_name)
        validate_args(a)
        out.append(a)
    return out


async def _run_policy(args, ps, parker: Parker, shared: dict):
    name = args.policy_name
    tracker = Tracker(args, stdout=ps.rank == 0)
    actor, critic, start = create_training_models(args, ps)
    rollout = create_rollout_components(args, ps, actor, tracker)
    rollout.executor.load(start - 1 if start > 0 else None)
    update_weights(args, actor, rollout)
    loop = asyncio.get_running_loop()
    for rollout_id in range(start, args.num_rollout):
        # generation and training are blocking calls: run them on the default executor so policies interleave
        pack = await loop.run_in_executor(None, rollout.executor.get, rollout_id)
        shard = object_store.get(pack.data_ref)
        metrics = {f"{name}/{k}": v for k, v in pack.metrics.items()}
        tm = await loop.run_in_executor(None, actor.train, rollout_id, shard)
        metrics.update({f"{name}/{k}": v for k, v in tm.items()})
        object_store.remove(pack.data_ref)
        update_weights(args, actor, rollout)
        shared.setdefault("history", {}).setdefault(name, []).append(metrics)
        if args.save and args.save_interval and (rollout_id + 1) % args.save_interval == 0:
            actor.save_model(rollout_id)
            # the set of checkpoints of one rollout id is complete only when every policy has written its own
            await parker.park(lambda rid=rollout_id: shared.setdefault("complete_saves", []).append(rid))
        tracker.log(metrics, rollout_id)
    parker.leave()
    tracker.finish()
    return name


async def train_multi_policy(policy_args: list):
    ps = create_parallel_state(policy_args[0])
    parker = Parker(len(policy_args))
    shared: dict = {}
    names = await asyncio.gather(*[_run_policy(a, ps, parker, shared) for a in policy_args])
    shared["policies"] = list(names)
    return shared


def main(argv=None):
    import sys

    argv = list(sys.argv[1:] if argv is None else argv)
    p = build_parser()
    p.add_argument("--multi-policy-config", required=True)
    pre, _ = p.parse_known_args([a for a in argv])
    common = parse_args([a for i, a in enumerate(argv) if a != "--multi-policy-config" and (i == 0 or argv[i - 1] != "--multi-policy-config")])
    return asyncio.run(train_multi_policy(load_policy_args(common, pre.multi_policy_config)))


if __name__ == "__main__":
    main()
