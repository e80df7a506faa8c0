"""Rollout engine on a GPU with layers of the benchmark's shape (hidden 2048, 32/4 heads of 128, 16 experts top-8,
full vocabulary): every decode batch bucket — with padding rows, routed-expert recording and CUDA graphs — must
sample in-range ids whose log-probs equal those of a plain full forward of prompt + output (training kernels)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _full_forward_logprobs(model, ids, dev):
    from miles_b200.models.qwen3 import ForwardMeta

    T = len(ids)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32, device=dev),
                       cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=dev), max_seqlen=T)
    with torch.no_grad():
        h = model(torch.tensor(ids, dtype=torch.int32, device=dev), meta)
        return torch.log_softmax(model.logits(h).float(), -1)


@pytest.fixture(scope="module")
def engine():
    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import get_config

    cfg = get_config("qwen3-30B-A3B").with_(num_experts=16, num_layers=2)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    return Engine(cfg, device=dev, dtype=torch.bfloat16, max_running_requests=64, max_context_len=512, num_blocks=256, seed=0)


@pytest.mark.parametrize("n_req", [1, 3, 7, 12, 20, 30, 44, 64])
def test_decode_buckets_match_full_forward(engine, n_req):
    cfg, dev = engine.cfg, engine.device
    g = torch.Generator().manual_seed(100 + n_req)
    prompts = [torch.randint(3, cfg.vocab_size, (int(torch.randint(5, 150, (1,), generator=g)),), generator=g).tolist()
               for _ in range(n_req)]
    new = 5
    outs = engine.generate(prompts, {"temperature": 1.0, "max_new_tokens": new}, return_routed_experts=True)
    worst, total, cnt = 0.0, 0.0, 0
    for i in range(0, n_req, max(1, n_req // 6)):          # check a spread of rows against the full forward
        p, o = prompts[i], outs[i]
        ids = o["output_ids"]
        assert len(ids) == new and all(0 <= t < cfg.vocab_size for t in ids)
        lp = _full_forward_logprobs(engine.model, p + ids, dev)
        for j, (t, (got, tid, _)) in enumerate(zip(ids, o["meta_info"]["output_token_logprobs"])):
            assert tid == t and got == got
            d = abs(float(lp[len(p) + j - 1, t]) - got)
            worst, total, cnt = max(worst, d), total + d, cnt + 1
    # a near-tie in the router may pick another expert on one path: allow single outliers, keep the mean tight
    assert total / cnt < 0.03 and worst < 0.6, (n_req, total / cnt, worst)


def test_decode_while_batch_drains(engine):
    """Requests of different lengths finish one after another: the runner passes through the smaller buckets with holes
    and compaction, and every sampled id stays in range with a finite log-prob."""
    cfg = engine.cfg
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(3, cfg.vocab_size, (20 + 3 * i,), generator=g).tolist() for i in range(40)]
    sps = [{"temperature": 1.0, "max_new_tokens": 2 + (i * 7) % 23} for i in range(40)]
    outs = engine.generate(prompts, sps, return_routed_experts=True)
    for sp, o in zip(sps, outs):
        assert len(o["output_ids"]) == sp["max_new_tokens"]
        assert all(0 <= t < cfg.vocab_size for t in o["output_ids"])
        assert all(lp == lp and lp <= 0.0 for lp, _, _ in o["meta_info"]["output_token_logprobs"])


@pytest.mark.parametrize("steps", [2, 4, 8])
def test_several_decode_steps_per_round_trip_give_the_same_samples(engine, steps):
    """Replaying the decode graph several times per host round trip (sampled token fed back on the device) must give
    exactly the tokens, log-probs and routed experts of one step per round trip: stop tokens, length limits that fall
    inside a round trip, block boundaries and rows that finish early included."""
    cfg = engine.cfg
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (5, 63, 64, 65, 120, 17, 33)]
    sps = [{"temperature": 1.0, "max_new_tokens": m, "seed": 50 + i, "stop_token_ids": list(range(0, cfg.vocab_size, 3)) if i % 2 else []}
           for i, m in enumerate((1, 2, 9, 70, 13, 40, 5))]
    res = {}
    for k in (1, steps):
        engine.decode_steps_per_sync = k
        engine.decode_steps_idle = 32 if k >= 4 else k      # 32: read back in chunks of 8 while the later steps run
        outs = engine.generate(prompts, [dict(sp) for sp in sps], return_routed_experts=True)
        res[k] = [(o["output_ids"], [round(x[0], 4) for x in o["meta_info"]["output_token_logprobs"]], o["meta_info"]["finish_reason"]["type"],
                   o["meta_info"].get("routed_experts")) for o in outs]
        assert engine._free_blocks() == engine.allocator.num_blocks if hasattr(engine.allocator, "num_blocks") else True
    engine.decode_steps_per_sync, engine.decode_steps_idle = 4, 32
    for a, b in zip(res[1], res[steps]):
        assert a[0] == b[0] and a[2] == b[2], (a[0], b[0], a[2], b[2])
        assert max((abs(x - y) for x, y in zip(a[1], b[1])), default=0.0) < 2e-3
        assert a[3] == b[3]
    assert any(r[2] == "stop" for r in res[1]) and any(r[2] == "length" for r in res[1])


@pytest.mark.gpu
def test_vmm_arena_pause_releases_memory_and_resume_restores_contents():
    """The trainer's sleep / wake-up mechanism: tagged arena regions give their physical pages back (device memory in use
    drops), keep their addresses, and come back with their contents."""
    from miles_b200.native import runtime as rt

    if not rt.available():
        pytest.skip("native runtime not built")
    arena = rt.VmmArena(torch.cuda.current_device())
    try:
        a = arena.empty((64 << 20,), torch.float32, tag="optimizer")        # 256 MB
        b = arena.empty((1 << 20,), torch.bfloat16, tag="other")
        a.copy_(torch.arange(a.numel(), device="cuda", dtype=torch.float32))
        b.fill_(3.0)
        torch.cuda.synchronize()
        ptr = a.data_ptr()
        free0, _ = torch.cuda.mem_get_info()
        released = arena.pause("optimizer", keep_contents=True)
        free1, _ = torch.cuda.mem_get_info()
        assert released >= a.numel() * 4 and free1 - free0 >= (200 << 20), (released, free1 - free0)
        assert float(b.float().sum()) == 3.0 * b.numel()                   # other tags stay mapped
        arena.resume("optimizer")
        free2, _ = torch.cuda.mem_get_info()
        assert free2 <= free1 - (200 << 20) and a.data_ptr() == ptr
        assert torch.equal(a[:1000], torch.arange(1000, device="cuda", dtype=torch.float32))
        assert float(a[-1]) == float(torch.tensor(a.numel() - 1, dtype=torch.float32))      # fp32 rounds 2^26 − 1 up
    finally:
        arena.close()


@pytest.mark.gpu
def test_trainer_sleep_uses_the_arena_and_training_continues():
    from miles_b200.args import parse_args
    from miles_b200.models.config import ModelConfig
    from miles_b200.native import runtime as rt
    from miles_b200.train.actor import TrainActor

    if not rt.available():
        pytest.skip("native runtime not built")
    cfg = ModelConfig(name="sleepy", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                      ffn_hidden_size=512)
    args = parse_args("--rollout-batch-size 2 --n-samples-per-prompt 2 --num-rollout 1 --lr 1e-3 --colocate --offload-train".split())
    actor = TrainActor(args, device="cuda:0")
    actor.init(cfg)
    assert actor.arena is not None
    d = actor.optimizer.domains[0]
    before = d.master.clone()
    free0, _ = torch.cuda.mem_get_info()
    actor.sleep()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 > free0
    actor.wake_up()
    assert torch.equal(d.master, before)


@pytest.mark.gpu
def test_prefix_cache_and_chunked_prefill_on_cuda():
    """Cached prefixes and chunked prompts on the CUDA engine (gathered keys + tcgen05 forward with separate key
    sequences) give the tokens of an engine that recomputes every prompt in one piece."""
    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import ModelConfig

    cfg = ModelConfig(name="pc-test", vocab_size=2048, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                      ffn_hidden_size=1024, max_position=4096)
    mk = lambda **kw: Engine(cfg, device="cuda", dtype=torch.bfloat16, num_blocks=96, block_size=64, seed=3, **kw)  # noqa: E731
    g = torch.Generator().manual_seed(1)
    base = torch.randint(3, 2000, (300,), generator=g).tolist()
    turn2 = base + torch.randint(3, 2000, (150,), generator=g).tolist()
    turn3 = turn2 + torch.randint(3, 2000, (700,), generator=g).tolist()
    sp = {"temperature": 0.0, "max_new_tokens": 8}
    plain, cached, chunked = mk(prefix_cache=False), mk(), mk(prefix_cache=False, chunked_prefill_size=256)
    for p in (base, turn2, turn3):
        a = plain.generate(p, dict(sp))
        b = cached.generate(p, dict(sp))
        c = chunked.generate(p, dict(sp))
        la, lb, lc = ([x[0] for x in o["meta_info"]["output_token_logprobs"]] for o in (a, b, c))
        # greedy tokens may flip where two logits tie within bf16 noise: compare log-probs of the common prefix
        n = next((i for i, (x, y, z) in enumerate(zip(a["output_ids"], b["output_ids"], c["output_ids"])) if not (x == y == z)), 8)
        assert n >= 1
        assert max(abs(x - y) for x, y in zip(la[:n], lb[:n])) < 5e-2 and max(abs(x - y) for x, y in zip(la[:n], lc[:n])) < 5e-2
    assert cached.stats["prefix_cache_hit_tokens"] == 256 + 448 and cached.stats["extend_tokens"] > 0
    assert chunked.stats["extend_tokens"] > 0


@pytest.mark.gpu
def test_cuda_ipc_bucket_between_processes(tmp_path):
    """An engine server in ANOTHER process on this GPU receives a bucket as a CUDA-IPC handle of the sender's flat buffer
    and ends up with bit-identical weights (no kernel of one process waits on the other: the copy is ordered by the HTTP
    request / response)."""
    import socket
    import subprocess
    import sys

    from miles_b200.engine.server import weight_checksums
    from miles_b200.models.config import PRESETS
    from miles_b200.models.convert import to_hf
    from miles_b200.models.qwen3 import build_model
    from miles_b200.orchestration.workers.fleet import RemoteEngine, wait_healthy
    from miles_b200.parallel.state import ParallelState

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = subprocess.Popen([sys.executable, "-m", "miles_b200.engine.server", "--model-name", "tiny", "--port", str(port),
                             "--mem-fraction-static", "0.05"], stdout=open(tmp_path / "server.log", "wb"), stderr=subprocess.STDOUT)
    try:
        try:
            wait_healthy(f"http://127.0.0.1:{port}", 240.0, alive=lambda: proc.poll() is None)
        except Exception as e:
            raise AssertionError(f"{e}\n--- server log ---\n" + open(tmp_path / "server.log", errors="replace").read()[-3000:])
        cfg = PRESETS["tiny"]
        model = build_model(cfg, ParallelState.single(), dtype=torch.bfloat16, device="cuda", seed=123)
        named = [x for n, p in model.named_parameters() for x in to_hf(n, p.data, cfg)]
        eng = RemoteEngine(f"http://127.0.0.1:{port}")
        nbytes = eng.update_weights_from_tensor(named, weight_version=5)
        assert nbytes >= sum(t.numel() * t.element_size() for _, t in named)
        out = eng._post("weights_checker", {"action": "compare", "checksums": weight_checksums(model)})
        assert out == {"success": True, "mismatched": []}, out
        eng._post("update_weight_version", {"weight_version": 5})
        assert eng.get_weight_version() == 5
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()


@pytest.mark.gpu
def test_output_top_logprobs_on_the_cuda_runner(engine):
    """Requests that ask for the k most likely tokens run their decode steps eagerly (the logits are read after the step);
    other requests of the same batch are unaffected and the reported log-prob of the sampled token is among / consistent
    with the top entries."""
    cfg = engine.cfg
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (17, 40)]
    a = engine.add_request(prompts[0], {"temperature": 0.0, "max_new_tokens": 5}, True, top_logprobs_num=3)
    b = engine.add_request(prompts[1], {"temperature": 0.0, "max_new_tokens": 5}, True)
    while not (a.finished and b.finished):
        engine.step()
    ra, rb = a.to_response(engine), b.to_response(engine)
    tops = ra["meta_info"]["output_top_logprobs"]
    assert len(tops) == 5 and "output_top_logprobs" not in rb["meta_info"]
    for (lp, tok, _), top in zip(ra["meta_info"]["output_token_logprobs"], tops):
        assert top[0][1] == tok and abs(top[0][0] - lp) < 2e-2 and top[0][0] >= top[1][0] >= top[2][0]
    assert len(rb["output_ids"]) == 5


@pytest.mark.gpu
def test_prefill_decode_disaggregation_on_cuda(engine):
    """The prompt's KV leaves one engine as a tensor and is stored into another engine's cache (on the last GPU of the box when
    there are several: one device-to-device copy); decoding there gives the first engine's tokens up to a near-tie flip and
    its log-probs on the common prefix."""
    import asyncio

    from miles_b200.engine.engine import Engine
    from miles_b200.engine.pd import PDClient

    cfg = engine.cfg
    dev = torch.device("cuda", torch.cuda.device_count() - 1)
    other = Engine(cfg, device=dev, dtype=torch.bfloat16, max_running_requests=16, max_context_len=512, num_blocks=128, seed=0)
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (40, 130, 65)]
    sp = {"temperature": 0.0, "max_new_tokens": 12}
    want = engine.generate(prompts, [dict(sp)] * 3, return_routed_experts=True)
    client = PDClient([engine], [other])

    async def run():
        outs = await asyncio.gather(*[client.generate({"input_ids": p, "sampling_params": dict(sp), "return_logprob": True,
                                                       "return_routed_experts": True}) for p in prompts])
        await client.finish()
        return outs

    got = asyncio.run(run())
    for w, o in zip(want, got):
        n = next((i for i, (x, y) in enumerate(zip(w["output_ids"], o["output_ids"])) if x != y), len(w["output_ids"]))
        assert n >= 1 and len(o["output_ids"]) == 12
        a, b = ([x[0] for x in r["meta_info"]["output_token_logprobs"]][:n] for r in (w, o))
        assert max(abs(x - y) for x, y in zip(a, b)) < 5e-2
    assert other.stats["received_kv_tokens"] == sum(map(len, prompts)) and other.stats["prefill_tokens"] == 0
    assert not engine.held_kv and other._free_blocks() == other.allocator.num_blocks


@pytest.mark.gpu
def test_precapture_fills_every_bucket_and_generation_is_unchanged(engine):
    """`DecodeRunner.precapture` records a graph for every batch bucket up to the row limit without touching any request;
    generating afterwards replays them and gives the tokens an engine without the call gives."""
    cfg = engine.cfg
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (9, 30, 50)]
    sp = {"temperature": 0.0, "max_new_tokens": 6}
    before = engine.generate(prompts, [dict(sp)] * 3)
    n_before = len(engine.runner.graphs)
    added = engine.runner.precapture(records=(True, False))
    from miles_b200.engine.decode_runner import BUCKETS

    want = {(b, r) for b in BUCKETS if b <= engine.runner.max_rows for r in (True, False)}
    assert want <= set(engine.runner.graphs) and added == len(engine.runner.graphs) - n_before
    assert engine.runner.precapture(records=(True, False)) == 0
    after = engine.generate(prompts, [dict(sp)] * 3)
    assert [o["output_ids"] for o in after] == [o["output_ids"] for o in before]
    assert engine._free_blocks() == engine.allocator.num_blocks
