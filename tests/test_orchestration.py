"""RPC transport, worker-pool planning, launch commands, true-on-policy contracts and the debug runner (CPU)."""
import time
from types import SimpleNamespace

import pytest

from miles_b200.orchestration.rpc import RemoteError, RpcClient, RpcServer
from miles_b200.orchestration.worker_spec import (CommandWorkerSpec, LocalLauncher, PortAllocator, SchedulingSpec, ServeWorkerSpec,
                                                  plan)


class _Target:
    def __init__(self):
        self.n = 0

    def add(self, a, b=1):
        self.n += a + b
        return {"n": self.n, "blob": b"\x00\x01"}

    def slow(self, s):
        time.sleep(s)
        return "done"

    def ping(self):
        return "pong"

    def boom(self):
        raise ValueError("bad input")


def test_rpc_roundtrip_errors_and_concurrency_groups():
    srv = RpcServer(_Target(), concurrency={"default": 1, "health": 2}, groups={"ping": "health"})
    port = srv.start()
    c = RpcClient(f"http://127.0.0.1:{port}")
    try:
        assert c.add(2, b=3) == {"n": 5, "blob": b"\x00\x01"}
        with pytest.raises(RemoteError) as e:
            c.boom()
        assert e.value.kind == "ValueError" and "bad input" in str(e.value) and "remote traceback" in str(e.value)
        with pytest.raises(RemoteError):
            c.nope()
        # a health probe is answered while the single default slot is busy
        import threading

        t = threading.Thread(target=lambda: c.slow(0.5))
        t.start()
        time.sleep(0.1)
        t0 = time.time()
        assert c.ping() == "pong" and time.time() - t0 < 0.3
        t.join()
    finally:
        srv.stop()


def test_plan_colocated_and_disaggregated():
    train = ServeWorkerSpec("trainer", "pkg.Trainer", SchedulingSpec(num_cells=2, workers_per_cell=2, gpus_per_worker=1), env={"NCCL_CUMEM_ENABLE": 0})
    eng = CommandWorkerSpec("engine", ["python", "-m", "miles_b200.engine.server", "--port", "{port}", "--tp", "{world_size}"],
                            SchedulingSpec(num_cells=2, workers_per_cell=1, gpus_per_worker=2), ports=["port", "nccl_port"])
    ws = plan([train, eng], {"node0": 8}, colocate=False, ports=PortAllocator(base=41000))
    tr = [w for w in ws if w.pool == "trainer"]
    en = [w for w in ws if w.pool == "engine"]
    assert [w.env["CUDA_VISIBLE_DEVICES"] for w in tr] == ["0", "1", "2", "3"]
    assert [w.env["CUDA_VISIBLE_DEVICES"] for w in en] == ["4,5", "6,7"]
    assert [(w.cell, w.rank) for w in tr] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert tr[0].env["MASTER_PORT"] != tr[2].env["MASTER_PORT"] and tr[0].env["MASTER_PORT"] == tr[1].env["MASTER_PORT"]
    assert tr[0].env["NCCL_CUMEM_ENABLE"] == "0"
    assert en[0].command[-3] == str(en[0].ports["port"]) and en[0].ports["port"] != en[1].ports["port"]
    assert len({p for w in ws for p in w.ports.values()}) == 4
    co = plan([train, eng], {"node0": 4}, colocate=True, ports=PortAllocator(base=42000))
    assert [w.env["CUDA_VISIBLE_DEVICES"] for w in co if w.pool == "engine"] == ["0,1", "2,3"]
    with pytest.raises(AssertionError):
        plan([train, eng], {"node0": 4}, colocate=False)
    desc = LocalLauncher().launch(ws, dry_run=True)
    assert desc[0]["cmd"][2] == "miles_b200.orchestration.worker_spec" and "--serve" in desc[0]["cmd"]


def test_launch_commands_and_recipe():
    from miles_b200.args import parse_args
    from miles_b200.utils import launch

    shape = launch.model_args("qwen3-30B-A3B")
    assert shape[shape.index("--num-experts") + 1] == "128" and "--qk-layernorm" in shape
    recipe = launch.qwen3_30b_a3b_recipe(8)
    a = parse_args(recipe + ["--num-rollout", "1", "--rm-type", "math"])
    assert a.tensor_model_parallel_size == 4 and a.expert_model_parallel_size == 4 and a.global_batch_size == 256
    cmd = launch.execute_train(recipe, launch.ExecuteTrainConfig(num_gpus=8, dry_run=True))
    assert cmd[1:3] == ["-m", "torch.distributed.run"] and "--nproc-per-node=8" in cmd and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
    one = launch.execute_train("--model-name tiny", launch.ExecuteTrainConfig(num_gpus=1, entry="train_async.py", dry_run=True))
    assert one[1].endswith("train_async.py") and one[2:] == ["--model-name", "tiny"]


def test_true_on_policy_contracts(monkeypatch):
    from miles_b200.utils import true_on_policy as top

    for k in ("MILES_SPLIT_K", "MILES_DECODE_SPLITS", "MILES_TC_ATTENTION"):
        monkeypatch.delenv(k, raising=False)
    args = SimpleNamespace(model_name="qwen3-30B-A3B", rollout_top_p=0.9, rollout_top_k=50, sequence_parallel=True, num_experts=128)
    names = top.apply(args)
    assert "routing_replay" in names and args.rollout_top_p == 1.0 and args.sequence_parallel is False and args.use_routing_replay
    import os

    assert os.environ["MILES_SPLIT_K"] == "0" and os.environ["MILES_DECODE_SPLITS"] == "1"
    dense = SimpleNamespace(model_name="qwen3-4B", num_experts=0)
    assert "routing_replay" not in top.apply(dense)
    top.verify([{"rollout/step": 0, "train/train_rollout_logprob_abs_diff": 0.0, "train/tis": 1.0}])
    with pytest.raises(AssertionError):
        top.verify([{"rollout/step": 3, "train/train_rollout_logprob_abs_diff": 1e-6}])


def test_debug_runner(tmp_path):
    import torch

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import PRESETS
    from miles_b200.utils import debug

    out = debug.main(["run", "--model-name", "tiny", "--fp32", "--cpu", "--tokens", "5,9,13,21,34", "--backward"])
    assert len(out["logprobs"]) == 4 and out["grad_norm"] > 0
    eng = Engine(PRESETS["tiny"], device="cpu", dtype=torch.float32, seed=0, num_blocks=64, block_size=4)
    r = eng.generate([5, 9, 13], {"temperature": 1.0, "max_new_tokens": 5, "seed": 1})
    sample = {"tokens": [5, 9, 13] + r["output_ids"], "response_length": 5, "index": 0,
              "rollout_log_probs": [p[0] for p in r["meta_info"]["output_token_logprobs"]]}
    dump = tmp_path / "dump.pt"
    torch.save({"rollout_id": 0, "samples": [[sample]]}, dump)
    cmp = debug.main(["compare", "--model-name", "tiny", "--fp32", "--cpu", "--rollout-dump", str(dump)])
    assert cmp["max_abs_diff"] < 1e-4


def test_inference_controller_config_framing_and_health():
    from miles_b200.orchestration.inference_controller import (InferenceController, ServerCell, engine_launch_cmd,
                                                               load_serving_config)
    from miles_b200.testing.mock_engine import MockEngine

    models = load_serving_config({"models": [
        {"name": "policy", "model_path": "/ckpt/policy", "server_groups": [
            {"worker_type": "prefill", "num_gpus": 2, "num_gpus_per_engine": 1, "overrides": {"mem_fraction_static": 0.6}},
            {"worker_type": "decode", "num_gpus": 4, "num_gpus_per_engine": 2},
            {"worker_type": "placeholder", "num_gpus": 2}]},
        {"name": "teacher", "update_weights": False}]})
    assert [g.num_engines for g in models[0].groups] == [2, 2, 0] and models[1].groups[0].worker_type == "regular"
    cmd = engine_launch_cmd(models[0], models[0].groups[0], port=30010)
    assert cmd[:5] == ["python", "-m", "miles_b200.engine.server", "--port", "30010"] and "--mem-fraction-static" in cmd
    assert cmd[cmd.index("--disaggregation-mode") + 1] == "prefill"
    with pytest.raises(ValueError):
        load_serving_config({"models": [{"name": "x", "server_groups": [{"worker_type": "prefill"}]}]})

    engines = [MockEngine(), MockEngine()]
    ok = {id(engines[0]): True, id(engines[1]): True}
    ctl = InferenceController([ServerCell(e, "policy", models[0].groups[1]) for e in engines], probe=lambda e: ok[id(e)],
                              health_threshold=2)
    targets = ctl.start_update_weights()
    assert len(targets) == 2 and ctl.lock.holder == "update_weights" and all(e.paused for e in engines)
    ctl.end_update_weights(5)
    assert ctl.weight_version == 5 and all(e.weight_version == 5 and not e.paused for e in engines)
    assert [c[0] for c in engines[0].calls] == ["pause_generation", "flush_cache", "update_weight_version", "continue_generation"]
    ctl.offload()
    assert all(c.state == "offloaded" for c in ctl.cells) and engines[0].calls[-1][0] == "release_memory_occupation"
    ctl.onload()
    assert all(c.state == "alive" for c in ctl.cells)
    ok[id(engines[1])] = False
    ctl.tick()
    assert ctl.tick()["policy#1"] == "unhealthy" and ctl.engines() == [engines[0]]
    ctl.start_update_weights()
    ctl.end_update_weights(6)                               # the quarantined engine misses version 6
    ok[id(engines[1])] = True
    assert ctl.tick()["policy#1"] == "stale" and ctl.stale_engines() == [engines[1]]
    ctl.mark_synced(engines[1])
    assert ctl.tick()["policy#1"] == "alive"
