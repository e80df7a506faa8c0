"""Audit trail, dashboard store / API, and the checkpoint-conversion tool chain (CPU)."""
import json
import os

import torch

from miles_b200.audit import events as A
from miles_b200.dashboard.server import DashboardBackend, GpuSampler, SeriesStore, build_app, scrape_prometheus
from miles_b200.models import convert as mc
from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import build_model
from miles_b200.parallel.state import ParallelState


def test_audit_rules(tmp_path):
    log = A.EventLogger(str(tmp_path), "trainer", 0)
    eng = A.EventLogger(str(tmp_path), "engine", 0)
    w = {"a": torch.ones(4), "b": torch.arange(3.0)}
    cs = A.combined_checksum(A.model_checksums(w.items()))
    log.log("weights_published", version=1, checksum=cs)
    eng.log("weights_received", version=1, checksum=cs, engine="e0")
    wit = A.DataWitness(log)
    ids = wit.allocate(0, 6)
    wit.consumed(0, 0, ids[:3], dp_rank=0)
    wit.consumed(0, 0, ids[3:], dp_rank=1)
    for r in (0, 1):
        log.log("replica_checksum", step=0, dp_rank=r, checksum="same")
    assert A.analyze(str(tmp_path)) == []
    # now break each rule
    w["a"][0] = 2
    eng.log("weights_received", version=1, checksum=A.combined_checksum(A.model_checksums(w.items())), engine="e1")
    log.log("replica_checksum", step=1, dp_rank=0, checksum="x")
    log.log("replica_checksum", step=1, dp_rank=1, checksum="y")
    wit.consumed(0, 1, [ids[0]])
    wit.allocate(1, 2)
    found = {(f["rule"], f["problem"]) for f in A.analyze(str(tmp_path))}
    assert ("weight_checksums", "engine weights differ from trainer") in found
    assert ("cross_replica", "replicas diverged") in found
    assert ("witness", "samples trained on more than once") in found and ("witness", "samples never trained on") in found
    assert A.tensor_checksum(torch.ones(3)) != A.tensor_checksum(torch.ones(3) * (1 + 1e-7))


def test_dashboard_store_api_and_sampler(tmp_path):
    from fastapi.testclient import TestClient

    store = SeriesStore(max_points=3, jsonl=str(tmp_path / "m.jsonl"))
    be = DashboardBackend(store)
    for step in range(5):
        be.log({"train/loss": 1.0 / (step + 1), "note": "text is skipped"}, step, "rollout/step")
    assert len(store.get("train/loss")) == 3 and store.get("train/loss")[-1] == (4.0, 0.2)
    other = SeriesStore()
    other.load_jsonl(str(tmp_path / "m.jsonl"))
    assert len(other.get("train/loss")) == 5
    with TestClient(build_app(store)) as c:
        assert c.get("/api/names", params={"prefix": "train/"}).json() == ["train/loss"]
        assert c.get("/api/series", params={"name": "train/loss", "last": 2}).json() == [[3.0, 0.25], [4.0, 0.2]]
        assert "<canvas" in c.get("/").text or "canvas" in c.get("/").text
        c.post("/api/log", json={"metrics": {"x": 1}, "step": 9})
        assert store.get("x") == [(9.0, 1.0)]

    class FakeNvml:                                       # the sampler only reads; a fake NVML stands in for the driver
        NVML_CLOCK_SM = 1

        def nvmlDeviceGetCount(self):
            return 2

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetUtilizationRates(self, h):
            return type("U", (), {"gpu": 50 + h})()

        def nvmlDeviceGetMemoryInfo(self, h):
            return type("M", (), {"used": 2 ** 31})()

        def nvmlDeviceGetClockInfo(self, h, k):
            return 1965

        def nvmlDeviceGetPowerUsage(self, h):
            return 700000

        def nvmlDeviceGetCurrentClocksThrottleReasons(self, h):
            return 4

    out = GpuSampler(store, nvml=FakeNvml()).sample_once()
    assert out["gpu1/util"] == 51 and out["gpu0/mem_used_gb"] == 2.0 and out["gpu0/power_w"] == 700.0
    assert scrape_prometheus("# HELP x\nengine_tokens_total 12\nq{a=\"b\"} 3.5\nbad line\n") == {"engine_tokens_total": 12.0, 'q{a="b"}': 3.5}


def test_convert_tool_chain(tmp_path):
    from miles_b200.checkpoint import hf_io, torch_dist
    from miles_b200.tools import convert as tool

    cfg = PRESETS["tiny"]
    model = build_model(cfg, ParallelState.single(), dtype=torch.bfloat16, device="cpu", seed=0)
    hf_dir = str(tmp_path / "hf")
    named = [x for n, p in model.named_parameters() for x in mc.to_hf(n, p.detach(), cfg)]
    hf_io.save_hf_sharded(hf_dir, [named], cfg, write=True)
    assert os.path.exists(os.path.join(hf_dir, "config.json"))
    # HF → torch_dist → HF is the identity on every tensor
    rel = tool.main(["hf-to-torch-dist", "--hf", hf_dir, "--out", str(tmp_path / "td")])
    assert torch_dist.is_torch_dist_dir(rel) and open(tmp_path / "td" / "latest_checkpointed_iteration.txt").read() == "release"
    tool.main(["torch-dist-to-hf", "--load", str(tmp_path / "td"), "--out", str(tmp_path / "hf2"), "--hf-config", hf_dir])
    a, b = hf_io.load_hf_dir(hf_dir), hf_io.load_hf_dir(str(tmp_path / "hf2"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    # quantised exports: payload + scale tensors, config gains a quantisation block; fp8 → bf16 comes back close
    tool.main(["hf-to-fp8", "--hf", hf_dir, "--out", str(tmp_path / "fp8")])
    q = hf_io.load_hf_dir(str(tmp_path / "fp8"))
    name = "model.layers.0.self_attn.o_proj.weight"
    assert q[name].dtype == torch.float8_e4m3fn and name + "_scale_inv" in q and q["model.norm.weight"].dtype == torch.bfloat16
    assert json.load(open(tmp_path / "fp8" / "config.json"))["quantization_config"]["quant_method"] == "fp8"
    tool.main(["fp8-to-bf16", "--hf", str(tmp_path / "fp8"), "--out", str(tmp_path / "bf16")])
    back = hf_io.load_hf_dir(str(tmp_path / "bf16"))
    assert set(back) == set(a) and "quantization_config" not in json.load(open(tmp_path / "bf16" / "config.json"))
    assert (back[name].float() - a[name].float()).abs().max() < 0.08 * a[name].float().abs().max()
    tool.main(["hf-to-mxfp8", "--hf", hf_dir, "--out", str(tmp_path / "mx")])
    assert hf_io.load_hf_dir(str(tmp_path / "mx"))[name + "_scale_inv"].dtype == torch.uint8
    tool.main(["hf-to-int4-qdq", "--hf", hf_dir, "--out", str(tmp_path / "i4")])
    i4 = hf_io.load_hf_dir(str(tmp_path / "i4"))[name]
    assert i4.dtype == torch.bfloat16 and i4.float().view(-1, 32).unique(dim=1).shape[1] <= 32
    tool.main(["hf-to-nvfp4-qdq", "--hf", hf_dir, "--out", str(tmp_path / "n4")])
    assert hf_io.load_hf_dir(str(tmp_path / "n4"))[name].shape == a[name].shape


def test_run_with_audit_dir_allocates_and_consumes_every_witness(tmp_path, tiny_args):
    """`train.py --audit-dir`: the rollout executor gives every sample a witness id, the trainer reports the ids it
    consumed, and the analyser finds every sample trained on exactly once; `--snapshot-dir` leaves an HF snapshot."""
    import train as train_entry
    from test_e2e import BASE
    from miles_b200.args import parse_args
    from miles_b200.audit import events

    args = parse_args((BASE + f" --audit-dir {tmp_path / 'audit'} --num-rollout 2 --snapshot-dir {tmp_path / 'snap'} "
                       "--true-on-policy-mode").split())
    assert args.true_on_policy_contracts and args.rollout_top_p == 1.0
    train_entry.train(args)
    ev = events.read_events(str(tmp_path / "audit"))
    kinds = {e["kind"] for e in ev}
    assert {"witness_allocated", "witness_consumed", "weights_published"} <= kinds
    assert events.rule_witness(ev) == []
    latest = (tmp_path / "snap" / "latest").read_text().strip()
    assert (tmp_path / "snap" / latest / "config.json").exists()


def test_train_profiler_writes_traces_for_the_selected_window(tmp_path):
    """`--use-pytorch-profiler --profile-target train_overall train_actor`: one trace per target for the step window."""
    import glob

    import train as train_entry
    from test_e2e import BASE
    from miles_b200.args import parse_args

    for target in ("train_overall", "train_log_probs"):
        args = parse_args((BASE + f" --num-rollout 3 --use-pytorch-profiler --profile-target {target} "
                           f"--profile-step-start 1 --profile-step-end 2 --tensorboard-dir {tmp_path}").split())
        train_entry.train(args)
        names = [p.rsplit("/", 1)[-1] for p in glob.glob(str(tmp_path / "*.json*"))]
        assert any(n.startswith(f"{target}_rank_0") for n in names), (target, names)


def test_reference_flag_surface_parses_and_wired_flags_act(tmp_path):
    """Every flag name of the reference's own parser is accepted; a handful of the wired ones are checked for effect."""
    import re

    import train as train_entry
    from test_e2e import BASE
    from miles_b200.args import build_parser, parse_args

    have = {s for a in build_parser()._actions for s in a.option_strings}
    for must in ("--start-rollout-id", "--eval-top-k", "--dumper-enable", "--opd-teacher-urls", "--mlflow-tracking-uri",
                 "--pause-generation-mode", "--session-server-port", "--ci-metric-checker-key", "--offload-train-target"):
        assert must in have, must
    # behaviour: stop after rollout 1 of 5, no optimizer updates, checkpoint with per-rank checksums, audit analysis at the end
    args = parse_args((BASE + f" --num-rollout 5 --debug-exit-after-rollout 1 --debug-disable-optimizer --save {tmp_path / 'ck'} "
                       f"--save-interval 1 --save-local-weight-checksum --enable-witness --audit-dir {tmp_path / 'au'} "
                       "--enable-event-analyzer").split())
    tr = train_entry.train(args)
    assert len(tr.history.rows) == 2 and tr.actor.global_step == 0
    assert all(g == 0.0 for g in tr.history.series("train/grad_norm"))
    assert list((tmp_path / "ck").rglob("weight_checksum_rank00000.json"))
    assert tr.findings == []
    # --start-rollout-id overrides the resume point; --reset-optimizer-states restarts Adam on the loaded weights
    args = parse_args((BASE + f" --num-rollout 4 --load {tmp_path / 'ck'} --start-rollout-id 3 --reset-optimizer-states").split())
    tr = train_entry.train(args)
    assert [r["rollout/step"] for r in tr.history.rows] == [3]


def test_dumper_phases_and_compare(tmp_path):
    """--dumper-enable with the three phase lists: trainer log-prob passes, train passes (with parameters and gradients)
    and the engine's forwards land in their own trees; the compare tool matches a tree with itself and flags a change."""
    import torch

    from test_e2e import BASE, _run
    from miles_b200.utils import dumper as D

    d = str(tmp_path / "dump")
    _run(f"--num-rollout 1 --dumper-enable --dumper-dir {d} --dumper-inference steps=2 --dumper-fwd-only filter=layers.0.|log_probs "
         f"--dumper-fwd-bwd max_numel=64")
    assert sorted(os.listdir(d)) == ["fwd_bwd", "fwd_only", "inference"]
    inf = os.path.join(d, "inference")
    assert sorted(os.listdir(inf)) == ["step00000", "step00001"]                       # steps=2
    names = {f.split("___", 1)[1] for f in os.listdir(os.path.join(d, "fwd_only", "step00000", "rank000"))}
    assert names == {"layers.0.out.pt", "layers.0.attn.out.pt", "layers.0.mlp.out.pt", "log_probs.pt"}
    fb = os.path.join(d, "fwd_bwd", "step00000", "rank000")
    files = os.listdir(fb)
    assert any("___grad.layers.0.attn.wqkv" in f for f in files) and any("___param.embed" in f for f in files)
    big = torch.load(os.path.join(fb, next(f for f in files if "___param.embed" in f)), weights_only=False)
    assert big["meta"]["sampled"] and big["value"].numel() <= 64 and big["meta"]["norm"] > 0
    assert all(r["status"] == "ok" for r in D.compare(inf, inf))
    # perturb one tensor of a copy
    import shutil

    other = str(tmp_path / "other")
    shutil.copytree(inf, other)
    victim = os.path.join(other, "step00001", "rank000", sorted(os.listdir(os.path.join(other, "step00001", "rank000")))[0])
    blob = torch.load(victim, weights_only=False)
    blob["value"] = blob["value"] * 1.5
    torch.save(blob, victim)
    rows = D.compare(inf, other)
    assert [r["status"] for r in rows].count("diff") == 1
    assert D.main(["compare", inf, other]) == 1 and D.main(["compare", inf, inf]) == 0
    assert D.DumperConfig.kv_to_dict(["max-numel=8", "enable=false"]) == {"max_numel": 8, "enable": False}


def test_dashboard_phases_advisories_and_sample_views(tmp_path):
    """A run with --dump-details --use-miles-dashboard leaves metrics, per-rank phase lanes and rollout dumps; the dashboard
    serves timeline, advisories and sample / token views from them."""
    from fastapi.testclient import TestClient

    from test_e2e import _run
    from miles_b200.dashboard import advisory, phases
    from miles_b200.dashboard.server import SeriesStore, build_app

    d = str(tmp_path / "dump")
    _run(f"--dump-details {d} --use-miles-dashboard --num-rollout 2")
    assert os.path.exists(os.path.join(d, "dashboard", "metrics.jsonl")) and os.path.exists(os.path.join(d, "train_data", "1_0.pt"))
    rows = phases.read_phases(d)
    names = {(r["role"], r["phase"]) for r in rows}
    assert {("actor", "actor_train"), ("actor", "log_probs"), ("rollout", "generate")} <= names
    util = phases.utilisation(rows)
    assert 0.0 <= util["actor:0"]["idle"] < 1.0 and util["actor:0"]["phases"]["actor_train"] > 0
    store = SeriesStore()
    store.load_jsonl(os.path.join(d, "dashboard", "metrics.jsonl"))
    app = TestClient(build_app(store, d))
    tl = app.get("/api/phases").json()
    assert "actor:0" in tl["lanes"] and tl["t1"] > tl["t0"]
    assert app.get("/api/rollouts").json() == [0, 1]
    ro = app.get("/api/rollout/1").json()
    assert ro["summary"]["samples"] == 32 and len(ro["samples"]) == 32 and ro["summary"]["groups"] == 8
    tv = app.get("/api/sample/1/0/1").json()
    assert tv["tokens"][0]["part"] == "prompt" and tv["tokens"][-1]["part"] == "response" and tv["tokens"][-1]["rollout_log_prob"] is not None
    assert "timeline" in app.get("/").text
    # advisories from hand-made signals: a stalled lane, uneven ranks, truncation, train / rollout mismatch
    fake = [{"rank": r, "role": "actor", "phase": "actor_train", "start": 0.0, "end": 10.0 + 10 * r, "rollout_id": 0} for r in (0, 1)]
    fake.append({"rank": 0, "role": "actor", "phase": "log_probs", "start": 400.0, "end": 410.0, "rollout_id": 1})
    st = SeriesStore()
    for i in range(5):
        st.add_many({"rollout/truncated_ratio": 0.5, "train/train_rollout_logprob_abs_diff": 0.2, "perf/rollout_time": 30.0, "perf/train_time": 5.0}, i)
    found = advisory.compute_advisories(st, fake, min_gap_s=60.0)
    titles = " | ".join(a["title"] for a in found)
    assert found[0]["severity"] == "alarm" and "recorded nothing" in titles and "differs by" in titles and "length limit" in titles
    assert "disagree on log-probs" in titles and "generation takes" in titles
    assert advisory.compute_advisories(SeriesStore(), []) == []
