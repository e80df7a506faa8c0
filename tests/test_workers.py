"""Worker layer: reconcile loops, providers, registration hub / reporter, the process manager with generations, the
supervisor, and an HTTP engine fleet that survives the loss of an engine process (CPU; failures are made on the host)."""
import asyncio
import os
import sys
import time

import pytest

from miles_b200.orchestration.worker_spec import CommandWorkerSpec, SchedulingSpec
from miles_b200.orchestration.workers.manager import StaleGeneration, WorkerManager
from miles_b200.orchestration.workers.provider import (CellInfo, LocalProcessProvider, StaticWorkerProvider, WorkerInfo,
                                                       parse_host_port)
from miles_b200.orchestration.workers.reconcile import (Delete, PollingReconcileLoop, ReconcileLoop, Replace, RetryScheduler,
                                                        Upsert, WorkQueue)
from miles_b200.orchestration.workers.registration import RegistrationHub, RegistrationReporter, cell_from_json, cell_to_json

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SLEEPER = [sys.executable, "-c", "import time; time.sleep(120)"]


def test_work_queue_holds_a_key_once_and_retry_backs_off():
    async def body():
        q = WorkQueue()
        for k in ("a", "b", "a", "a"):
            q.add(k)
        assert len(q) == 2 and await q.get() == "a" and await q.get() == "b"
        q.add("a")                                     # may wait again once taken
        assert await q.get() == "a"
        q.shutdown()
        assert await q.get() is None

    asyncio.run(body())
    now = [0.0]
    woke = []
    r = RetryScheduler(woke.append, base_delay=1.0, max_delay=5.0, clock=lambda: now[0])
    assert [r.note_failure("k") for _ in range(4)] == [1.0, 2.0, 4.0, 5.0]
    now[0] = 4.9
    assert r.release_due() == []
    now[0] = 5.0 + 4.0
    assert r.release_due() == ["k"] and woke == ["k"]
    r.note_success("k")
    assert r.note_failure("k") == 1.0


def test_reconcile_loop_is_level_triggered_and_retries():
    async def body():
        feed: asyncio.Queue = asyncio.Queue()
        opened = [0]

        async def source():
            opened[0] += 1
            yield Replace(({"key": "w0", "parent": "c0", "v": 1}, {"key": "w1", "parent": "c1", "v": 1}))
            while True:
                ev = await feed.get()
                if ev == "break":
                    raise ConnectionError("stream lost")
                yield ev

        seen, fail_once = [], {"c1"}

        async def reconcile(parent):
            objs = sorted(o["key"] + ":" + str(o["v"]) for o in loop.store.by_parent(parent))
            if parent in fail_once:
                fail_once.discard(parent)
                raise RuntimeError("first try fails")
            seen.append((parent, tuple(objs)))

        loop = ReconcileLoop(source, reconcile, failure_base_delay=0.05, source_retry_delay=0.05, resync_period=None)
        async with loop:
            await asyncio.sleep(0.4)
            assert ("c0", ("w0:1",)) in seen and ("c1", ("w1:1",)) in seen            # c1 after one retry
            assert loop.stats["failed"] == 1
            n = len(seen)
            await feed.put(Upsert({"key": "w0", "parent": "c0", "v": 1}))           # unchanged object: nothing to do
            await feed.put(Upsert({"key": "w2", "parent": "c0", "v": 1}))
            await feed.put(Upsert({"key": "w2", "parent": "c0", "v": 2}))
            await feed.put(Delete("w1"))
            await asyncio.sleep(0.3)
            new = seen[n:]
            assert new[-1][0] in ("c0", "c1") and ("c0", ("w0:1", "w2:2")) in new and ("c1", ()) in new
            await feed.put("break")                                                 # the stream dies and is reopened with a Replace
            await asyncio.sleep(0.3)
            assert opened[0] == 2
            assert ("c0", ("w0:1",)) == [s for s in seen if s[0] == "c0"][-1]        # w2 is not in the reopened world

    asyncio.run(body())


def test_polling_loop_diffs_listings():
    async def body():
        world = {"a": 1, "b": 1}
        calls = []

        async def list_cells():
            return dict(world)

        async def reconcile(cid, info):
            if cid == "b" and info == 2 and ("b", 2) not in calls:
                calls.append((cid, info))
                raise RuntimeError("try again")
            calls.append((cid, info))

        loop = PollingReconcileLoop(list_cells, interval=0.05)
        stop = await loop.start(reconcile)
        assert calls == [("a", 1), ("b", 1)]
        world["b"] = 2
        del world["a"]
        await asyncio.sleep(0.3)
        await stop()
        assert calls[2:] == [("a", None), ("b", 2), ("b", 2)]                       # the failed cell is retried, the rest is not repeated

    asyncio.run(body())


def test_registration_hub_and_reporter():
    w = WorkerInfo("engine-c0-w0", "engine", "engine-c0", 0, 3, "10.0.0.5", (("port", 30000),))
    c = CellInfo("engine-c0", "engine", 3, True, (w,))
    assert cell_from_json(cell_to_json(c)) == c
    now = [0.0]
    hub = RegistrationHub(ttl=10.0, clock=lambda: now[0])
    assert hub.ingest({"reporter_id": "node-a", "seq": 2, "cells": [cell_to_json(c)]})
    assert not hub.ingest({"reporter_id": "node-a", "seq": 1, "cells": []})          # delayed older snapshot
    with pytest.raises(ValueError):
        hub.ingest({"reporter_id": "node-b", "seq": 1, "cells": [cell_to_json(c)]})  # a cell has one reporter
    assert list(asyncio.run(hub.list_cells())) == ["engine-c0"]
    now[0] = 11.0
    assert asyncio.run(hub.list_cells()) == {} and hub.reporters == {}               # silent reporter dropped with its cells

    async def body():
        hub2 = RegistrationHub(ttl=5.0)
        prov = StaticWorkerProvider("engine", ["127.0.0.1:1", "127.0.0.1:2"], probe=lambda h, p: p == 1)

        async def post(snap):
            hub2.ingest(snap)

        rep = RegistrationReporter("node-a", prov, post, interval=0.1, debounce=0.01)
        t = asyncio.ensure_future(rep.run(watch_interval=0.05))
        await asyncio.sleep(0.35)
        t.cancel()
        await asyncio.gather(t, return_exceptions=True)
        cells = await hub2.list_cells()
        assert {k: v.alive for k, v in cells.items()} == {"engine-c0": True, "engine-c1": False}
        assert rep.sent >= 2                                                         # heartbeats go on without changes

    asyncio.run(body())
    assert parse_host_port("http://h:81/") == ("h", 81)


def test_manager_generations_and_host_fault_injection(tmp_path):
    m = WorkerManager(log_dir=str(tmp_path))
    plan = m.launch([CommandWorkerSpec("sleeper", SLEEPER, SchedulingSpec(2, 2, 0), ports=["port"])])
    try:
        assert [p["name"] for p in plan] == ["sleeper-c0-w0", "sleeper-c0-w1", "sleeper-c1-w0", "sleeper-c1-w1"]
        cells = m.get_cell_infos()
        assert all(c.alive and c.generation == 0 and len(c.workers) == 2 for c in cells.values())
        assert len({w.port() for c in cells.values() for w in c.workers}) == 4
        m.inject_fault("sleeper-c1", mode="kill", worker_in_cell_index=1)
        assert m.wait_exit("sleeper-c1", 5.0)
        cells = m.get_cell_infos()
        assert cells["sleeper-c0"].alive and not cells["sleeper-c1"].alive             # one lost worker = a dead cell
        old = cells["sleeper-c1"].workers[0]
        new = m.restart_cell("sleeper-c1")
        assert new.alive and new.generation == 1 and new.workers[0].pid != old.pid
        with pytest.raises(StaleGeneration):
            m.get_worker("sleeper-c1-w0", expected_generation=0)
        assert m.get_worker("sleeper-c1-w0", expected_generation=1).generation == 1
        assert asyncio.run(LocalProcessProvider(m).list_cells())["sleeper-c1"].generation == 1
        assert os.path.exists(os.path.join(tmp_path, "sleeper-c1-w0.g1.log"))
    finally:
        m.stop_all()
    assert not any(c.alive for c in m.get_cell_infos().values())


def test_supervisor_ends_the_group_when_one_rank_fails():
    from miles_b200.orchestration.workers.supervisor import exit_code_of, supervise

    code = "import os,sys,time; r=int(os.environ['RANK']); assert os.environ['WORLD_SIZE']=='3'; sys.exit(7) if r==1 else time.sleep(60)"
    t0 = time.monotonic()
    assert supervise([sys.executable, "-c", code], 3, grace=5.0) == 7
    assert time.monotonic() - t0 < 30
    assert supervise([sys.executable, "-c", "pass"], 2) == 0
    assert exit_code_of(-9) == 137


def test_engine_fleet_survives_a_lost_engine(tmp_path):
    """Two engine servers + router launched as worker processes; the trainer pushes weights through the disk protocol;
    one engine process is killed on the host; the watcher restarts it under generation 1 and the next update re-syncs it."""
    sys.path.insert(0, ROOT)
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_training_models,
                                                 update_weights)

    args = parse_args(("--model-name tiny --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 6 "
                       "--num-rollout 2 --rm-type even_fraction --lr 1e-4 --advantage-estimator grpo "
                       "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 4 6 "
                       "--rollout-engine http --worker-provider local --rollout-num-engines 2 "
                       f"--update-weight-transfer-mode disk --update-weight-disk-dir {tmp_path}/sync --worker-log-dir {tmp_path}/logs").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    rollout = create_rollout_components(args, ps, actor)
    fleet = rollout.fleet
    try:
        assert len(rollout.engines) == 2 and fleet.router_url
        update_weights(args, actor, rollout)
        v1 = actor.weight_version
        assert [e.get_weight_version() for e in rollout.engines] == [v1, v1]
        from miles_b200.utils import object_store

        pack = rollout.executor.get(0)
        actor.train(0, object_store.get(pack.data_ref))
        fleet.manager.inject_fault("engine-c0", mode="kill")
        end = time.monotonic() + 240
        while not any(ev[0] == "restarted" for ev in fleet.events) and time.monotonic() < end:
            time.sleep(0.5)
        assert ("restarted", "engine-c0", 1) in fleet.events, (fleet.events, fleet.manager.log_tail("engine-c0-w0"))
        assert rollout.controller.stale_engines() == [fleet.engines["engine-c0"]]
        assert fleet.engines["engine-c0"].get_weight_version() == 0                     # fresh process, fresh weights
        update_weights(args, actor, rollout)
        assert [e.get_weight_version() for e in rollout.engines] == [actor.weight_version] * 2
        assert rollout.controller.stale_engines() == []
        # the tensor protocol towards engines in other processes: flat buckets (bytes here; CUDA-IPC handles on a GPU)
        from miles_b200.weight_update.updater import WeightUpdater

        for p in actor.model.parameters():
            p.data.add_(0.01)
        actor.weight_version += 1
        upd = WeightUpdater(args, actor, rollout.engines, mode="tensor")
        update_weights(args, actor, rollout, updater=upd)
        assert [e.get_weight_version() for e in rollout.engines] == [actor.weight_version] * 2
        from miles_b200.engine.server import weight_checksums

        want = weight_checksums(actor.model)
        for e in rollout.engines:                                                       # every tensor arrived bit-exactly
            assert e._post("weights_checker", {"action": "compare", "checksums": want}) == {"success": True, "mismatched": []}
        pack = rollout.executor.get(1)                                                  # both engines serve again
        assert len(object_store.get(pack.data_ref)["tokens"]) == 8
    finally:
        fleet.shutdown()


def test_registration_hub_over_http():
    import socket

    import requests

    from miles_b200.orchestration.workers.registration import http_poster

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    hub = RegistrationHub(ttl=30.0)
    server, thread = hub.serve(port=port)
    try:
        w = WorkerInfo("engine-c0-w0", "engine", "engine-c0", 0, 0, "127.0.0.1", (("port", 30000),))
        snap = {"reporter_id": "node-a", "seq": 1, "cells": [cell_to_json(CellInfo("engine-c0", "engine", 0, True, (w,)))]}
        out = asyncio.run(http_poster(f"http://127.0.0.1:{port}")(snap))
        assert out == {"accepted": True, "reporters": 1}
        cells = requests.get(f"http://127.0.0.1:{port}/cells").json()["cells"]
        assert cells[0]["workers"][0]["name"] == "engine-c0-w0"
        bad = {"reporter_id": "node-b", "seq": 1, "cells": [dict(snap["cells"][0])]}
        assert requests.post(f"http://127.0.0.1:{port}/register", json=bad).status_code == 422     # the cell has a reporter already
    finally:
        server.should_exit = True
        thread.join(5)


def test_trainer_pool_runs_grpo_ranks_under_the_worker_manager(tmp_path):
    """The trainer as a pool of supervised processes (no torchrun): two gloo ranks get their rendezvous variables from the
    planner, train two rollouts and exit 0; a rank that fails ends the pool with its exit code."""
    from miles_b200.utils.launch import ExecuteTrainConfig, execute_train

    args = ("--model-name tiny --fp32 --rollout-batch-size 8 --n-samples-per-prompt 4 --rollout-max-response-len 8 --num-rollout 2 "
            "--rm-type even_fraction --lr 1e-4 --colocate --advantage-estimator grpo "
            "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 6 10")
    cfg = ExecuteTrainConfig(num_gpus=2, launcher="workers", log_dir=str(tmp_path / "logs"), env={"CUDA_VISIBLE_DEVICES": ""})
    plan = execute_train(args, ExecuteTrainConfig(num_gpus=2, launcher="workers", dry_run=True))
    assert [p["env"]["RANK"] for p in plan] == ["0", "1"] and all(p["env"]["WORLD_SIZE"] == "2" for p in plan)
    assert plan[0]["env"]["MASTER_PORT"] == plan[1]["env"]["MASTER_PORT"] and plan[0]["cmd"][1].endswith("train.py")
    assert execute_train(args, cfg) == 0
    logs = sorted(os.listdir(tmp_path / "logs"))
    assert logs == ["trainer-0-0.g0.log", "trainer-0-1.g0.log"] or len(logs) == 2, logs
    text = open(tmp_path / "logs" / logs[0]).read()
    assert "rollout/step=1" in text
    bad = ExecuteTrainConfig(num_gpus=2, launcher="workers", log_dir=str(tmp_path / "bad"), env={"CUDA_VISIBLE_DEVICES": ""})
    assert execute_train(args + " --no-such-flag", bad) != 0


def test_engine_fleet_in_prefill_decode_roles(tmp_path):
    """`--rollout-pd-prefill-engines 1` over a fleet of two engine servers: rollouts go prompt → engine 0 → KV → engine 1, the
    trainer's recomputed log-probs equal the fleet's (the hand-over loses nothing), and the decode engine ran no prompt."""
    sys.path.insert(0, ROOT)
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_training_models,
                                                 update_weights)
    from miles_b200.utils import object_store

    args = parse_args(("--model-name tiny --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 6 "
                       "--num-rollout 1 --rm-type even_fraction --lr 1e-4 --advantage-estimator grpo "
                       "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 20 30 "
                       "--rollout-engine http --worker-provider local --rollout-num-engines 2 --rollout-pd-prefill-engines 1 "
                       f"--update-weight-transfer-mode disk --update-weight-disk-dir {tmp_path}/sync --worker-log-dir {tmp_path}/logs").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    rollout = create_rollout_components(args, ps, actor)
    try:
        update_weights(args, actor, rollout)
        pack = rollout.executor.get(0)
        shard = object_store.get(pack.data_ref)
        assert len(shard["tokens"]) == 8 and all(r == 6 for r in shard["response_lengths"])
        m = actor.train(0, shard)
        assert m["train/train_rollout_logprob_abs_diff"] < 1e-4, m["train/train_rollout_logprob_abs_diff"]
    finally:
        rollout.fleet.shutdown()


def test_serving_config_sizes_the_fleet_and_assigns_roles(tmp_path):
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import apply_serving_config

    cfg = tmp_path / "serve.yaml"
    cfg.write_text("models:\n  - name: judge\n    eval_only: true\n    server_groups: [{worker_type: regular, num_gpus: 1}]\n"
                   "  - name: policy\n    model_path: /models/policy\n    server_groups:\n"
                   "      - {worker_type: prefill, num_gpus: 1}\n      - {worker_type: decode, num_gpus: 3}\n")
    args = parse_args(f"--model-name tiny --rollout-engine http --worker-provider local --engine-config {cfg}".split())
    apply_serving_config(args)
    assert (args.rollout_num_engines, args.rollout_pd_prefill_engines, args.hf_checkpoint) == (4, 1, "/models/policy")
    cfg.write_text("models:\n  - name: policy\n    server_groups: [{worker_type: regular, num_gpus: 2}]\n")
    args = parse_args(f"--model-name tiny --rollout-engine http --worker-provider local --sglang-config {cfg}".split())
    apply_serving_config(args)
    assert (args.rollout_num_engines, args.rollout_pd_prefill_engines) == (2, 0)
    cfg.write_text("models:\n  - name: policy\n    server_groups: [{worker_type: regular, num_gpus: 4, num_gpus_per_engine: 2}]\n")
    args = parse_args(f"--model-name tiny --engine-config {cfg}".split())
    apply_serving_config(args)
    assert (args.rollout_num_engines, args.rollout_num_gpus_per_engine) == (2, 2)
    cfg.write_text("models:\n  - name: policy\n    server_groups: [{worker_type: prefill, num_gpus: 2, num_gpus_per_engine: 2}, "
                   "{worker_type: decode, num_gpus: 2, num_gpus_per_engine: 2}]\n")
    with pytest.raises(AssertionError):
        apply_serving_config(parse_args(f"--model-name tiny --engine-config {cfg}".split()))


def test_engine_fleet_with_a_two_rank_engine(tmp_path):
    """`--rollout-num-gpus-per-engine 2`: the fleet's engine is a cell of two ranks (experts sharded) behind one port; weights
    arrive through the disk protocol on both ranks and a rollout through it matches the trainer's log-probs."""
    sys.path.insert(0, ROOT)
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_training_models,
                                                 update_weights)
    from miles_b200.utils import object_store

    args = parse_args(("--model-name tiny-moe --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 6 "
                       "--num-rollout 1 --rm-type even_fraction --lr 1e-4 --advantage-estimator grpo "
                       "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 8 12 "
                       "--rollout-engine http --worker-provider local --rollout-num-engines 1 --rollout-num-gpus-per-engine 2 "
                       f"--update-weight-transfer-mode disk --update-weight-disk-dir {tmp_path}/sync --worker-log-dir {tmp_path}/logs").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    for p in actor.model.parameters():                      # the engine starts from its own random weights: make ours differ
        p.data.mul_(1.01)
    rollout = create_rollout_components(args, ps, actor)
    try:
        assert len(rollout.fleet.manager.cells["engine-c0"].workers) == 2
        update_weights(args, actor, rollout)
        time.sleep(0.5)                                     # the load is applied by the engine's next control tick
        shard = object_store.get(rollout.executor.get(0).data_ref)
        m = actor.train(0, shard)
        assert len(shard["tokens"]) == 8 and m["train/train_rollout_logprob_abs_diff"] < 1e-4, m["train/train_rollout_logprob_abs_diff"]
    finally:
        rollout.fleet.shutdown()


def test_kubernetes_provider_maps_pods_to_cells(tmp_path):
    """The pod list of a `kubectl`-shaped command becomes cells: labels give pool / cell / worker / generation, the named
    container port and the pod IP give the address, a cell is alive only when every pod is Running and ready."""
    import json
    import stat

    from miles_b200.orchestration.workers.kubernetes import KubernetesWorkerProvider

    def pod(name, ip, phase="Running", ready=True, labels=None, restarts=0, deleting=False):
        meta = {"name": name, "labels": labels or {}}
        if deleting:
            meta["deletionTimestamp"] = "2026-01-01T00:00:00Z"
        return {"metadata": meta, "spec": {"containers": [{"ports": [{"name": "metrics", "containerPort": 9000}, {"name": "http", "containerPort": 30000}]}]},
                "status": {"phase": phase, "podIP": ip, "containerStatuses": [{"ready": ready, "restartCount": restarts}]}}

    items = [pod("eng-a", "10.0.0.1", labels={"miles/cell": "0", "miles/worker": "0"}),
             pod("eng-b", "10.0.0.2", labels={"miles/cell": "0", "miles/worker": "1"}, restarts=2),
             pod("eng-c", "10.0.0.3", labels={"miles/cell": "1"}, ready=False),
             pod("eng-d", "10.0.0.4", labels={"miles/cell": "2", "miles/generation": "7"}),
             pod("eng-e", "10.0.0.5", labels={"miles/cell": "3"}, deleting=True)]
    data = tmp_path / "pods.json"
    data.write_text(json.dumps({"items": items}))
    fake = tmp_path / "kubectl"
    fake.write_text(f"#!/bin/sh\ncase \"$*\" in *'-l app=engine'*'-n rl'*) cat {data};; *) echo bad args: $* >&2; exit 3;; esac\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    prov = KubernetesWorkerProvider("engine", "app=engine", namespace="rl", kubectl=str(fake))
    cells = asyncio.run(prov.list_cells())
    assert sorted(cells) == ["engine-c0", "engine-c1", "engine-c2", "engine-c3"]
    c0 = cells["engine-c0"]
    assert c0.alive and c0.generation == 2 and [w.url() for w in c0.workers] == ["http://10.0.0.1:30000", "http://10.0.0.2:30000"]
    assert not cells["engine-c1"].alive and cells["engine-c2"].generation == 7 and not cells["engine-c3"].alive
    assert asyncio.run(prov.get_addrs("engine-c2-w0")).host == "10.0.0.4"
    bad = KubernetesWorkerProvider("engine", "app=other", kubectl=str(fake))
    with pytest.raises(RuntimeError):
        asyncio.run(bad.list_cells())
