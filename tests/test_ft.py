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
