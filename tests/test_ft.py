"""Fault tolerance on the host: cells and controller, heartbeats, engine health, fault injector, the deterministic
in-process group, the mock engine, in-memory checkpoints and their transfer, and the reconfigurable cross-cell gradient
all-reduce with a rank that leaves between steps (CPU ranks over gloo; no GPU is involved)."""
import os
import sys
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import _free_port, run_distributed  # noqa: E402

from miles_b200.ft.checkpoint_transfer import InMemoryCheckpoint, build_manifest, rebuild  # noqa: E402
from miles_b200.ft.controller import (Cell, CellController, CellState, EngineHealthChecker, HeartbeatMonitor,  # noqa: E402
                                      MiniFTController)
from miles_b200.testing.det_pg import LocalWorld  # noqa: E402
from miles_b200.testing.fault_injector import FaultInjector, InjectedFault, parse_rules  # noqa: E402
from miles_b200.testing.mock_engine import MockEngine  # noqa: E402


class _Worker:
    def __init__(self, fail_on=None):
        self.fail_on, self.calls, self.killed, self.state = fail_on, [], False, 0

    def init(self):
        self.calls.append("init")

    def train(self, step):
        if self.fail_on == step:
            raise RuntimeError("boom")
        self.state += 1
        return self.state

    def kill(self):
        self.killed = True


def test_cell_controller_retries_on_quorum_and_heals():
    workers = {i: _Worker(fail_on=2 if i == 1 else None) for i in range(3)}
    cells = [Cell(i, [workers[i]]) for i in range(3)]
    published = []
    ctl = CellController(cells, min_quorum=2, on_membership=published.append)
    ctl.execute("init")
    assert all(c.state == CellState.ALIVE for c in cells)
    assert set(ctl.execute("train", 1)) == {0, 1, 2}
    out = ctl.execute("train", 2)                       # cell 1 fails, is fenced, the step re-runs on {0, 2}
    assert set(out) == {0, 2} and cells[1].state == CellState.ERRORED and workers[1].killed
    assert published[-1] == [0, 2]
    moved = []
    ctl.heal(1, [_Worker()], transfer=lambda donor, healed: moved.append((donor.cell_id, healed.cell_id)))
    assert cells[1].state == CellState.ALIVE and cells[1].generation == 1 and moved == [(0, 1)]
    assert published[-1] == [0, 1, 2]
    with pytest.raises(RuntimeError):
        CellController([Cell(0, [_Worker(fail_on=0)])], min_quorum=1).execute("train", 0)


def test_heartbeats_and_mini_controller():
    now = [0.0]
    store = {}

    class DictStore:
        def set(self, k, v):
            store[k] = v

        def get(self, k):
            return store[k]

    mon = HeartbeatMonitor(DictStore(), timeout_s=5.0, clock=lambda: now[0])
    cells = [Cell(i, [_Worker()]) for i in range(2)]
    ctl = CellController(cells)
    ctl.execute("init")
    ft = MiniFTController(ctl, mon, worker_to_cell={"w0": 0, "w1": 1})
    mon.beat("w0")
    mon.beat("w1")
    assert ft.tick()["fenced"] == []
    now[0] = 4.0
    mon.beat("w0")
    now[0] = 7.0                                        # w1 last beat at t=0: dead; w0 at t=4: alive
    assert mon.dead() == ["w1"]
    r = ft.tick()
    assert r["fenced"] == [1] and r["alive"] == [0]
    ft.register_replacement(1, [_Worker()])
    assert ft.tick()["healed"] == [1] and cells[1].state == CellState.ALIVE


def test_engine_health_checker_quarantine_and_recovery():
    engines = ["a", "b"]
    ok = {"a": True, "b": False}
    events = []
    hc = EngineHealthChecker(engines, probe=lambda e: ok[e], threshold=2, on_unhealthy=lambda e: events.append(("down", e)),
                             on_recovered=lambda e: events.append(("up", e)))
    hc.check_once()
    assert hc.healthy() == ["a", "b"]
    hc.check_once()
    assert hc.healthy() == ["a"] and events == [("down", "b")]
    ok["b"] = True
    hc.check_once()
    assert hc.healthy() == ["a", "b"] and events[-1] == ("up", "b")


def test_fault_injector_rules():
    fi = FaultInjector(rank=1, rules=parse_rules("rank=1,step=3,point=before_allreduce,kind=raise;rank=0,step=3,kind=raise"))
    fi.at("before_allreduce", step=2)
    with pytest.raises(InjectedFault):
        fi.at("before_allreduce", step=3)
    fi.at("before_allreduce", step=3)                    # once
    fi.inject("drop", point="heartbeat", step=5)
    assert not fi.should_drop("heartbeat", 4) and fi.should_drop("heartbeat", 5) and not fi.should_drop("heartbeat", 5)
    fi.inject("error_code", point="launch", arg=700)
    assert fi.error_code("launch") == 700 and fi.error_code("launch") == 0
    t0 = time.time()
    fi.inject("sleep", point="slow", arg=0.05)
    fi.at("slow")
    assert time.time() - t0 >= 0.05


def test_local_world_collectives_are_deterministic():
    def body(pg):
        x = torch.tensor([0.1 * (pg.rank + 1), 1e8 if pg.rank == 2 else 0.0])
        s = pg.all_reduce(x.clone())
        g = pg.all_gather(torch.tensor([pg.rank]))
        a2a = pg.all_to_all([torch.tensor([pg.rank * 10 + j]) for j in range(pg.world_size)])
        b = pg.broadcast_object({"v": pg.rank}, src=3)
        return s, [int(t) for t in g], [int(t) for t in a2a], b

    r1 = LocalWorld(4).run(body)
    r2 = LocalWorld(4).run(body)
    assert all(torch.equal(a[0], b[0]) for a, b in zip(r1, r2))
    assert r1[1][1] == [0, 1, 2, 3] and r1[2][2] == [2, 12, 22, 32] and r1[0][3] == {"v": 3}
    with pytest.raises(ValueError):
        LocalWorld(2).run(lambda pg: (_ for _ in ()).throw(ValueError("x")) if pg.rank == 1 else pg.barrier())


def test_mock_engine_session_frame_and_versions():
    eng = MockEngine(tokens_per_step=2)
    r = eng.add_request([5, 6, 7], {"max_new_tokens": 6})
    eng.step()
    eng.pause_generation("retract")
    assert eng.step() is False
    eng.flush_cache()
    eng.update_weight_version(4)
    eng.continue_generation()
    while not r.done.is_set():
        eng.step()
    out = r.to_response(eng)
    assert len(out["output_ids"]) == 6 and out["meta_info"]["weight_version_spans"] == [[0, 2], [4, 4]]
    assert [c[0] for c in eng.calls] == ["pause_generation", "flush_cache", "update_weight_version", "continue_generation"]
    again = MockEngine(tokens_per_step=2).generate([5, 6, 7], {"max_new_tokens": 6})
    assert again["output_ids"] == out["output_ids"]      # deterministic in the prompt


def test_in_memory_checkpoint_and_dedup_manifest():
    flat = torch.arange(12, dtype=torch.float32)
    state = {"model": {"a": flat[:4], "b": flat[4:].view(2, 4)}, "optimizer": {"state": {0: {"m": torch.ones(3)}}, "step": 7},
             "names": ["x", "y"]}
    manifest, bufs = build_manifest(state)
    assert len(bufs) == 2                                # a and b share one storage: sent once
    back = rebuild(manifest, [b.clone() for b in bufs])
    assert torch.equal(back["model"]["b"], state["model"]["b"]) and back["optimizer"]["step"] == 7
    assert torch.equal(back["optimizer"]["state"][0]["m"], torch.ones(3)) and back["names"] == ["x", "y"]
    ck = InMemoryCheckpoint()
    ck.save(state, 3)
    flat.add_(100)
    st, step = ck.load()
    assert step == 3 and float(st["model"]["a"][1]) == 1.0


# ---- gloo ranks ----------------------------------------------------------------------------------------------------

def _transfer_body(rank, world):
    from miles_b200.ft.checkpoint_transfer import recv_state, send_state

    if rank == 0:
        flat = torch.arange(10, dtype=torch.float32)
        n = send_state({"w": flat[:6].view(2, 3), "v": flat[6:], "meta": {"step": 5}}, dst=1)
        assert n == 40
    else:
        st = recv_state(src=0)
        assert st["meta"]["step"] == 5 and st["w"].tolist() == [[0, 1, 2], [3, 4, 5]] and st["v"].tolist() == [6, 7, 8, 9]


def test_checkpoint_transfer_between_ranks():
    run_distributed(_transfer_body, 2)


def _indep_dp_body(rank, world, port):
    """Three single-rank cells average gradients; cell 2 leaves between steps 1 and 2 (host-side exit from the loop),
    the controller (cell 0 here) publishes the new membership, the survivors rebuild the group and carry on."""
    from miles_b200.ft.indep_dp import IndepDP
    from miles_b200.testing.fault_injector import FaultInjector, InjectedFault

    comm = IndepDP(rank, "127.0.0.1", port, timeout_s=5.0, is_store_master=(rank == 0))
    if rank == 0:
        comm.members.publish(0, [0, 1, 2])
    else:
        time.sleep(0.3)
    comm.follow_membership()
    fi = FaultInjector(rank=rank)
    fi.inject("raise", rank=2, step=2, point="between_steps")
    for step in range(4):
        try:
            fi.at("between_steps", step)
        except InjectedFault:
            comm.members.report_dead(rank)                # the leaving rank says so on the host, then stops
            return
        if rank == 0 and step == 2:
            while not comm.members.is_dead(2):
                time.sleep(0.01)
            comm.members.publish(1, [0, 1])
        if step == 2 and rank == 1:
            while comm.members.current()[0] != 1:
                time.sleep(0.01)
        comm.follow_membership()
        g = [torch.full((4,), float(rank + 1) * (step + 1))]
        committed, cells = comm.step(g)
        want = sum((c + 1) * (step + 1) for c in cells) / len(cells)
        assert committed and torch.allclose(g[0], torch.full((4,), want))
        assert cells == ([0, 1, 2] if step < 2 else [0, 1])
    assert comm.consensus(rank == 0) is False             # one cell vetoes → nobody commits


def test_indep_dp_reconfigures_when_a_cell_leaves():
    run_distributed(_indep_dp_body, 3, (_free_port(),), timeout=120)


def test_train_py_retries_a_failed_trainer_call_under_fault_tolerance(monkeypatch):
    """`--use-fault-tolerance`: the driver's trainer handle is a CellController; a step that raises once is retried and the
    run completes with the same number of optimizer steps."""
    import train as train_entry
    from test_e2e import BASE
    from miles_b200.args import parse_args
    from miles_b200.train.actor import TrainActor

    calls = {"n": 0}
    real = TrainActor.train

    def flaky(self, rollout_id, shard):
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("injected host-side failure")
        return real(self, rollout_id, shard)

    monkeypatch.setattr(TrainActor, "train", flaky)
    args = parse_args((BASE + " --use-fault-tolerance --num-rollout 2").split())
    tr = train_entry.train(args)
    assert calls["n"] == 3 and len(tr.history.rows) == 2
    assert tr.actor.global_step == 2


# ---- cell REST API + the in-job controller loop ---------------------------------------------------------------------

def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_cell_api_lists_fences_and_heals():
    import types

    import requests

    from miles_b200.ft.api_server import MiniFTController, http_cell_client, start_api_server
    from miles_b200.ft.controller import Cell, CellController
    from miles_b200.orchestration.inference_controller import InferenceController, ServerCell, ServerGroup

    class W:
        def __init__(self):
            self.fail = False

        def init(self):
            return "ok"

        def train(self, step):
            if self.fail:
                raise RuntimeError("host-side failure")
            return step

    class Eng:
        def __init__(self):
            self.ok, self.version, self.paused = True, 0, False

        def pause_generation(self, mode="retract"):
            self.paused = True

        def continue_generation(self):
            self.paused = False

        def get_weight_version(self):
            return self.version

    workers = [W(), W()]
    cells = CellController([Cell(0, [workers[0]]), Cell(1, [workers[1]])], min_quorum=1)
    cells.execute("init")
    trainer = types.SimpleNamespace(cells=cells)
    engines = [Eng(), Eng()]
    group = ServerGroup("regular", 1, 1)
    ictl = InferenceController([ServerCell(e, "default", group) for e in engines], probe=lambda e: e.ok, health_threshold=1)
    rollout = types.SimpleNamespace(controller=ictl, fleet=None)
    port = _free_port()
    server, thread, _ = start_api_server(types.SimpleNamespace(api_server_port=port, api_server_host="127.0.0.1"), trainer, rollout)
    base = f"http://127.0.0.1:{port}/api/v1"
    try:
        assert requests.get(f"{base}/health").json() == {"status": "ok"}
        items = requests.get(f"{base}/cells").json()["items"]
        assert [c["metadata"]["name"] for c in items] == ["trainer-0", "trainer-1", "rollout-0", "rollout-1"]
        assert all(c["status"]["phase"] == "Running" for c in items)
        r = requests.get(f"{base}/cells/nope")
        assert r.status_code == 404 and r.json()["reason"] == "NotFound" and r.json()["kind"] == "Status"
        assert requests.patch(f"{base}/cells/trainer-1", json={"spec": {"pause": True}}).status_code == 400
        # a trainer cell fails on the host → the API shows it, the controller loop fences and later heals it
        workers[1].fail = True
        cells.execute("train", 1)                                  # retried on the quorum (cell 0)
        c1 = requests.get(f"{base}/cells/trainer-1").json()
        assert c1["status"]["phase"] == "Failed" and c1["status"]["conditions"][1]["status"] == "False"
        now = [0.0]
        get_cells, patch = http_cell_client(f"http://127.0.0.1:{port}")
        ft = MiniFTController(get_cells, patch, resume_delay=5.0, clock=lambda: now[0])
        ft.poll_and_heal()
        assert ft.log == [("suspended", "trainer-1", 5.0)]
        assert requests.get(f"{base}/cells/trainer-1").json()["spec"]["suspend"] is True
        now[0] = 4.0
        ft.poll_and_heal()                                         # still fenced: the delay has not passed
        assert len(ft.log) == 1
        workers[1].fail = False
        now[0] = 5.5
        ft.poll_and_heal()
        assert ft.log[-1] == ("resumed", "trainer-1")
        c1 = requests.get(f"{base}/cells/trainer-1").json()
        assert c1["status"]["phase"] == "Running" and c1["status"]["generation"] == 1 and not c1["spec"]["suspend"]
        assert sorted(cells.execute("train", 2)) == [0, 1]
        # rollout cells: a failed probe shows as unhealthy; suspend pauses the engine; resume re-admits it as stale when it
        # missed a weight update
        engines[0].ok = False
        ictl.tick()
        assert requests.get(f"{base}/cells/rollout-0").json()["status"]["phase"] == "Failed"
        ictl.weight_version = 3
        engines[0].ok = True
        requests.patch(f"{base}/cells/rollout-0", json={"spec": {"suspend": True}})
        assert engines[0].paused
        out = requests.patch(f"{base}/cells/rollout-0", json={"spec": {"suspend": False}}).json()
        assert out["status"]["phase"] == "Running" and not engines[0].paused and ictl.stale_engines() == [engines[0]]
        # fault injection is refused where there is no process of ours to signal
        r = requests.post(f"{base}/cells/rollout-1/inject-fault", json={"mode": "kill"})
        assert r.status_code == 400 and r.json()["reason"] == "BadRequest"
        # second consecutive failure of the same cell doubles the fence time
        workers[1].fail = True
        cells.execute("train", 3)
        ft.poll_and_heal()
        assert ft.log[-1] == ("suspended", "trainer-1", 10.0)
    finally:
        server.should_exit = True
        thread.join(5)


def test_api_fault_injection_makes_the_next_train_call_raise_and_retry(tmp_path):
    """inject-fault (mode raise) on the trainer cell of this process: the next train call raises on the host before any
    launch, the fault-tolerant handle rolls back and retries, the step completes."""
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import requests

    from test_e2e import BASE
    from miles_b200.args import parse_args
    from miles_b200.ft.api_server import start_api_server
    from miles_b200.orchestration.wiring import (create_parallel_state, create_rollout_components, create_trainer_controller,
                                                 create_training_models)
    from miles_b200.testing import fault_injector
    from miles_b200.utils import object_store

    port = _free_port()
    args = parse_args((BASE + f" --use-fault-tolerance --api-server-port {port}").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    trainer = create_trainer_controller(args, actor)
    rollout = create_rollout_components(args, ps, actor)
    server, thread, _ = start_api_server(args, trainer, rollout)
    try:
        r = requests.post(f"http://127.0.0.1:{port}/api/v1/cells/trainer-0/inject-fault", json={"mode": "raise"})
        assert r.status_code == 200
        pack = rollout.executor.get(0)
        out = trainer.train(0, object_store.get(pack.data_ref))
        assert out["train/grad_norm"] > 0
        assert ("raise", "train", 0) in fault_injector.GLOBAL.log
        kinds = [k for k, _ in trainer.cells.log]
        assert "cell_failed" in kinds and "healed" in kinds
    finally:
        server.should_exit = True
        thread.join(5)
