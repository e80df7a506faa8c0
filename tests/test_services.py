"""Session server (token-in-token-out chat), Tinker-style multi-LoRA service, multi-policy training, delta weight
transfer and snapshot publishing — all on the CPU engine."""
import asyncio
import os
from types import SimpleNamespace

import pytest
import torch

from miles_b200.engine.engine import Engine
from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import build_model
from miles_b200.parallel.state import ParallelState
from miles_b200.rollout.client import InProcEngineClient
from miles_b200.session.core import SessionManager
from miles_b200.session.tito import ByteChatTokenizer, TitoTokenizer


def _engine(model=None):
    return Engine(PRESETS["tiny"], model=model, device="cpu", dtype=torch.float32, seed=0, num_blocks=256, block_size=8,
                  eos_token_ids=[257])


def test_tito_incremental_ids_are_a_pure_append():
    tok = ByteChatTokenizer()
    tito = TitoTokenizer(tok)
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"}]
    start = tito.start(msgs)
    assert tok.decode(start).endswith("<|im_start|>assistant\n")
    gen = tok("4")["input_ids"] + [257]                             # model wrote "4<|im_end|>"
    close = tito.close_assistant_turn(gen)
    assert tok.decode(close) == "\n"
    assert tito.close_assistant_turn(tok("4")["input_ids"]) == tok("<|im_end|>\n")["input_ids"]
    traj = start + gen + close
    prev = msgs + [{"role": "assistant", "content": "4"}]
    ext = tito.extend(prev, [{"role": "tool", "content": "ok"}])
    full = tok(tito.render(prev + [{"role": "tool", "content": "ok"}], add_generation_prompt=True))["input_ids"]
    assert traj + ext == full                                        # same ids as a fresh render, earlier ids untouched


def test_session_manager_keeps_exact_trajectory_and_forks():
    eng = _engine()
    client = InProcEngineClient([eng])
    mgr = SessionManager(ByteChatTokenizer(), client.generate, default_sampling={"temperature": 0.0, "max_new_tokens": 6})

    async def go():
        await client.begin()
        s = mgr.create("ep1")
        m1 = [{"role": "user", "content": "hi"}]
        r1 = await mgr.chat("ep1", m1)
        m2 = m1 + [r1["choices"][0]["message"], {"role": "user", "content": "more"}]
        r2 = await mgr.chat("ep1", m2)
        # a request that rewrites the first user turn forks a branch instead of corrupting the stored one
        r3 = await mgr.chat("ep1", [{"role": "user", "content": "different"}])
        await client.finish()
        return s, r1, r2, r3

    s, r1, r2, r3 = asyncio.run(go())
    t = s.trajectory()
    assert t["response_length"] == len(t["loss_mask"]) == len(t["rollout_log_probs"])
    assert sum(t["loss_mask"]) == r1["usage"]["completion_tokens"] + r2["usage"]["completion_tokens"]
    # masked-in positions are exactly what greedy decoding of the stored prefix yields: the engine saw these very ids
    P = t["prompt_length"]
    first_gen = t["tokens"][P:P + r1["usage"]["completion_tokens"]]
    again = eng.generate(t["tokens"][:P], {"temperature": 0.0, "max_new_tokens": 6})["output_ids"]
    assert again == first_gen
    assert r3["session_id"] != "ep1" and mgr.get(r3["session_id"]).parent == "ep1"
    sample = mgr.to_sample("ep1")
    assert sample.response_length == t["response_length"] and sample.loss_mask == t["loss_mask"]


def _lora_model(slots=3):
    from miles_b200.train import lora

    cfg = PRESETS["tiny"]
    model = build_model(cfg, ParallelState.single(), dtype=torch.float32, device="cpu", seed=0)
    args = SimpleNamespace(lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, lora_target_modules=["wqkv", "wo", "w13", "w2"],
                           lora_num_slots=slots, lora_adapter_path=None, seed=0, model_name="tiny")
    lora.apply_lora(model, args)
    return model, args


def _datum(tokens, weights=None):
    d = {"model_input": {"chunks": [{"tokens": tokens[:-1]}]}, "loss_fn_inputs": {"target_tokens": tokens[1:]}}
    if weights is not None:
        d["loss_fn_inputs"]["weights"] = weights
    return d


def test_tinker_service_trains_tenants_independently(tmp_path):
    from miles_b200.tinker.service import TinkerService

    model, args = _lora_model()
    eng = _engine(model)
    svc = TinkerService(model, args, engine=eng)
    a, b = svc.create_model("tenant-a"), svc.create_model("tenant-b")
    assert (a.slot, b.slot) == (0, 1) and svc.capabilities()["free_slots"] == 1
    data = [_datum([5, 9, 13, 21, 34, 55]), _datum([7, 7, 8, 9])]
    base = svc.forward("tenant-a", data)
    l0 = base["metrics"]["loss:sum"]
    for _ in range(8):
        svc.forward_backward("tenant-a", data, "cross_entropy")
        st = svc.optim_step("tenant-a", {"learning_rate": 5e-2})
    assert st["metrics"]["step"] == 8 and st["metrics"]["grad_norm"] > 0
    assert svc.forward("tenant-a", data)["metrics"]["loss:sum"] < l0 - 0.05      # tenant a learned
    assert abs(svc.forward("tenant-b", data)["metrics"]["loss:sum"] - l0) < 1e-4  # tenant b is untouched
    # importance-sampling loss with per-token advantages runs and produces per-datum log-probs
    lp = base["loss_fn_outputs"][0]["logprobs"]
    d = _datum([5, 9, 13, 21, 34, 55])
    d["loss_fn_inputs"].update(logprobs=lp, advantages=[1.0] * len(lp))
    out = svc.forward_backward("tenant-b", [d], "importance_sampling")
    assert len(out["loss_fn_outputs"][0]["logprobs"]) == 5
    # sampling uses the tenant's adapter; the base model (no tenant) differs from tenant a after training
    sp = {"temperature": 0.0, "max_tokens": 5}
    sa = svc.sample("tenant-a", [5, 9, 13], sp)["sequences"][0]
    s0 = svc.sample(None, [5, 9, 13], sp)["sequences"][0]
    assert len(sa["tokens"]) == 5 and len(s0["tokens"]) == 5
    # save → unload → new tenant in the recycled slot starts from zero → load restores
    svc.save_weights("tenant-a", str(tmp_path / "a"), export_peft=True)
    assert os.path.exists(tmp_path / "a" / "peft" / "adapter_config.json")
    la = svc.forward("tenant-a", data)["metrics"]["loss:sum"]
    svc.unload_model("tenant-a")
    svc.create_model("filler")                          # takes the never-used slot; tenant c gets the recycled one
    c = svc.create_model("tenant-c")
    assert c.slot == 0 and abs(svc.forward("tenant-c", data)["metrics"]["loss:sum"] - l0) < 1e-4
    svc.load_weights("tenant-c", str(tmp_path / "a"))
    assert abs(svc.forward("tenant-c", data)["metrics"]["loss:sum"] - la) < 1e-4
    fid = svc.submit(svc.optim_step, "nobody")
    assert svc.retrieve(fid)["status"] == "error" and svc.retrieve(fid)["status"] == "unknown"


def test_tinker_http_roundtrip():
    from fastapi.testclient import TestClient

    from miles_b200.tinker.server import build_app
    from miles_b200.tinker.service import TinkerService

    model, args = _lora_model(2)
    svc = TinkerService(model, args, engine=_engine(model))
    with TestClient(build_app(svc)) as c:
        assert c.get("/api/v1/healthz").json()["status"] == "ok"
        mid = c.post("/api/v1/create_model", json={"lora_config": {"rank": 4}}).json()["model_id"]
        rid = c.post("/api/v1/forward_backward", json={"model_id": mid, "forward_backward_input": {
            "data": [_datum([3, 4, 5, 6])], "loss_fn": "cross_entropy"}}).json()["request_id"]
        out = c.post("/api/v1/retrieve_future", json={"request_id": rid}).json()
        assert len(out["loss_fn_outputs"][0]["logprobs"]) == 3
        rid = c.post("/api/v1/optim_step", json={"model_id": mid, "adam_params": {"learning_rate": 1e-3}}).json()["request_id"]
        assert c.post("/api/v1/retrieve_future", json={"request_id": rid}).json()["metrics"]["step"] == 1
        rid = c.post("/api/v1/asample", json={"model_id": mid, "prompt": {"tokens": [3, 4]}, "sampling_params": {"max_tokens": 3}}).json()["request_id"]
        assert len(c.post("/api/v1/retrieve_future", json={"request_id": rid}).json()["sequences"][0]["tokens"]) == 3
        assert c.post("/api/v1/create_model", json={"lora_config": {"rank": 64}}).status_code == 409


def test_parker_and_multi_policy(tmp_path):
    import yaml

    import train_multi_policy as TMP
    from miles_b200.args import parse_args

    async def barrier_demo():
        p, order = TMP.Parker(3), []

        async def task(i):
            await asyncio.sleep(0.01 * i)
            await p.park(lambda: order.append("leader"))
            order.append(i)

        await asyncio.gather(*[task(i) for i in range(3)])
        return order, p.passes

    order, passes = asyncio.run(barrier_demo())
    assert order[0] == "leader" and sorted(order[1:]) == [0, 1, 2] and passes == 1
    cfg = tmp_path / "policies.yaml"
    cfg.write_text(yaml.safe_dump([{"name": "small_lr", "overrides": {"lr": 1e-5}}, {"name": "big_lr", "overrides": {"lr": 1e-3, "seed": 7}}]))
    common = parse_args(("--model-name tiny --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 6 "
                         "--num-rollout 2 --rm-type even_fraction --colocate --data-source-path miles_b200.rollout.data_source.SyntheticSource "
                         f"--synthetic-prompt-len 4 6 --save {tmp_path / 'ck'} --save-interval 1").split())
    shared = asyncio.run(TMP.train_multi_policy(TMP.load_policy_args(common, str(cfg))))
    assert sorted(shared["policies"]) == ["big_lr", "small_lr"] and shared["complete_saves"] == [0, 1]
    assert len(shared["history"]["small_lr"]) == 2 and os.path.isdir(tmp_path / "ck" / "big_lr")


def test_native_codecs_xxh64_and_zero_run_length_delta():
    """XXH64 against the algorithm's published vectors; the byte-plane + zero-run-length coder round-trips (with and without
    a base, every element size, empty and incompressible inputs) and rejects damaged streams without writing out of range."""
    import numpy as np

    from miles_b200.native import runtime as rt

    rt.build()
    assert rt.xxh64(b"") == 0xEF46DB3751D8E999 and rt.xxh64(b"abc") == 0x44BC2CF5AD770999
    assert rt.xxh64(b"a" * 100, 7) != rt.xxh64(b"a" * 100, 8) and rt.xxh64(np.arange(64, dtype=np.uint8)) == rt.xxh64(bytes(range(64)))
    rng = np.random.default_rng(0)
    for elem in (1, 2, 4, 8):
        base = rng.integers(0, 256, 4096 * elem, dtype=np.uint8)
        cur = base.copy()
        idx = rng.choice(cur.size // elem, 300, replace=False) * elem          # a few low bytes change
        cur[idx] ^= rng.integers(1, 256, idx.size, dtype=np.uint8)
        enc = rt.delta_encode(cur, base, elem)
        assert len(enc) < cur.size // 4 and (rt.delta_decode(enc, cur.size, base) == cur).all()
        plain = rt.delta_encode(cur, None, elem)                                 # no base: random bytes do not shrink
        assert len(plain) <= cur.size + cur.size // 64 + 64 and (rt.delta_decode(plain, cur.size) == cur).all()
        bad = bytearray(enc)
        bad[len(bad) // 2] ^= 0xFF
        try:
            out = rt.delta_decode(bytes(bad), cur.size, base)                    # either rejected or a different, in-range result
            assert out.size == cur.size
        except ValueError:
            pass
        with pytest.raises(ValueError):
            rt.delta_decode(enc[: len(enc) // 2], cur.size, base)
    assert rt.delta_decode(rt.delta_encode(np.zeros(0, np.uint8)), 0).size == 0
    z = np.zeros(1 << 16, np.uint8)
    assert len(rt.delta_encode(z, z, 2)) < 32


@pytest.mark.parametrize("codec", ["auto", "zrle", "zlib"])
def test_delta_writer_reader_and_snapshots(tmp_path, codec):
    from miles_b200.weight_update.delta import DeltaReader, DeltaWriter, SnapshotPublisher

    torch.manual_seed(0)
    w = {"a.weight": torch.randn(64, 32).bfloat16(), "b.weight": torch.randn(16).float()}
    wr = DeltaWriter(str(tmp_path / "d"), full_every=3, codec=codec)
    rd = DeltaReader(str(tmp_path / "d"))
    infos = []
    for v in range(1, 6):
        w = {k: (t.float() + 1e-3 * torch.randn_like(t.float()) * (k == "a.weight")).to(t.dtype) for k, t in w.items()}
        infos.append(wr.publish(v, w.items()))
        if v in (2, 5):                                   # the reader skips versions and walks the chain
            st = rd.update_to()
            assert rd.version == v and all(torch.equal(st[k], w[k]) for k in w)
    assert [i["full"] for i in infos] == [True, False, False, True, False]
    assert infos[1]["stored_bytes"] < infos[0]["stored_bytes"]     # unchanged tensor + sparse XOR compress well
    fresh = DeltaReader(str(tmp_path / "d"))
    assert all(torch.equal(fresh.update_to(5)[k], w[k]) for k in w)
    blob = tmp_path / "d" / "v5" / "t00000.bin"
    blob.write_bytes(b"\x00" + blob.read_bytes()[1:])
    with pytest.raises(Exception):
        DeltaReader(str(tmp_path / "d")).update_to(5)
    cfg = PRESETS["tiny"]
    model = build_model(cfg, ParallelState.single(), dtype=torch.float32, device="cpu", seed=0)
    from miles_b200.models.convert import to_hf

    def buckets():
        yield [x for n, p in model.named_parameters() for x in to_hf(n, p.detach(), cfg)]

    pub = SnapshotPublisher(str(tmp_path / "snap"), cfg, every=2, keep=1)
    assert pub.maybe_publish(1, buckets()) is None
    for step in (2, 4):
        assert pub.maybe_publish(step, buckets()).endswith(f"step_{step}")
    assert open(tmp_path / "snap" / "latest").read() == "step_4"
    assert sorted(x for x in os.listdir(tmp_path / "snap") if x.startswith("step_")) == ["step_4"]
    from miles_b200.checkpoint import hf_io

    assert "model.embed_tokens.weight" in hf_io.load_hf_dir(str(tmp_path / "snap" / "step_4"))


# ---- chat families of the token-in-token-out tokenizer --------------------------------------------------------------

FAMILY_SPECIALS = {
    "qwen3": ["<|im_start|>", "<|im_end|>", "<|endoftext|>"],
    "glm47": ["[gMASK]", "<sop>", "<|system|>", "<|user|>", "<|assistant|>", "<|observation|>", "<|endoftext|>"],
    "deepseek": ["<｜begin▁of▁sentence｜>", "<｜User｜>", "<｜Assistant｜>", "<｜tool▁output▁begin｜>", "<｜tool▁output▁end｜>", "<｜end▁of▁sentence｜>"],
    "kimi": ["<|im_system|>", "<|im_user|>", "<|im_assistant|>", "<|im_middle|>", "<|im_end|>"],
    "llama": ["<|begin_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"],
    "gemma": ["<bos>", "<start_of_turn>", "<end_of_turn>"],
}


@pytest.mark.parametrize("family", sorted(FAMILY_SPECIALS))
def test_tito_family_trajectory_equals_full_render(family):
    """For every family: start → model turn (ends the way that family's models end a turn) → appended tool + user
    messages → the kept trajectory equals the tokenisation of the fully rendered conversation, the model's ids untouched."""
    from miles_b200.session.tito import ByteChatTokenizer, TitoTokenizer
    from miles_b200.session.tito_families import guess_family

    tok = ByteChatTokenizer(FAMILY_SPECIALS[family])
    assert guess_family(tok) == family
    tito = TitoTokenizer(tok, family)
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"}]
    ids = tito.start(msgs)
    assert ids == tito.encode(tito.render(msgs, add_generation_prompt=True))
    answer = tito.encode("it is 4")
    if family == "glm47":
        gen = answer + tito.encode("<|observation|>")        # GLM ends its turn by sampling the next role tag
    else:
        gen = answer + tito.encode(tito.spec.eot)
    traj = ids + gen + tito.close_assistant_turn(gen)
    history = msgs + [{"role": "assistant", "content": "it is 4"}]
    new = [{"role": "tool", "content": "calc says 4"}, {"role": "user", "content": "thanks, and 3+3?"}]
    traj = traj + tito.extend(history, new, pretokenized=traj)
    want = tito.encode(tito.render(history + new, add_generation_prompt=True))
    assert traj == want, (tito.decode(traj), tito.decode(want))
    assert traj[len(ids):len(ids) + len(answer)] == answer
    rep = tito.check_against_fresh(history + new, traj[:-len(tito.encode(tito.spec.generation_prompt))])
    assert rep["special_equal"] and rep["equal"]
    with pytest.raises(ValueError):
        tito.extend(history, [{"role": "assistant", "content": "x"}])          # an assistant message cannot be injected


def test_tito_qwen_tools_thinking_and_grouped_tool_results():
    from miles_b200.session.tito import ByteChatTokenizer, TitoTokenizer
    from miles_b200.session.tito_families import QWEN3, QWEN35, compare_token_sequences

    tools = [{"type": "function", "function": {"name": "add", "parameters": {"type": "object"}}}]
    msgs = [{"role": "user", "content": "add"},
            {"role": "assistant", "content": "", "reasoning_content": "need the tool",
             "tool_calls": [{"function": {"name": "add", "arguments": "{\"a\": 1}"}}]},
            {"role": "tool", "content": "1"}, {"role": "tool", "content": "2"}]
    text = QWEN3.render(msgs, add_generation_prompt=True, tools=tools, enable_thinking=False)
    assert "<tools>\n" + '{"type": "function"' in text and "# Tools" in text
    assert '<think>\nneed the tool</think>\n<tool_call>\n{"name": "add", "arguments": {"a": 1}}\n</tool_call><|im_end|>' in text
    assert "<|im_start|>user\n<tool_response>\n1\n</tool_response>\n<tool_response>\n2\n</tool_response><|im_end|>" in text   # one turn
    assert text.endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert "<function=add>\n<parameter=a>\n1\n</parameter>" in QWEN35.render(msgs)
    t = TitoTokenizer(ByteChatTokenizer(), "qwen3")
    assert (t.reasoning_parser, t.tool_call_parser) == ("qwen3", "qwen25")
    rep = compare_token_sequences([1, 256, 5, 257, 10], [1, 256, 6, 7, 257], {256, 257}, {10})
    assert not rep["equal"] and rep["special_equal"] and rep["first_diff"] == 2
    assert not compare_token_sequences([256, 257], [256], {256, 257})["special_equal"]


def test_session_server_with_family_and_sample_picking():
    import asyncio
    import types

    from miles_b200.session.core import SessionManager, drop_same_prompt_retries, session_samples
    from miles_b200.session.tito import ByteChatTokenizer
    from miles_b200.types import Sample

    tok = ByteChatTokenizer(FAMILY_SPECIALS["glm47"])

    async def generate(payload):
        reply = list(b"ok") + [tok.SPECIALS["<|user|>"]]
        return {"text": "", "meta_info": {"output_token_logprobs": [[-0.5, t] for t in reply], "finish_reason": {"type": "stop"}}}

    m = SessionManager(tok, generate, family="glm47")
    s = m.create("a")
    out = asyncio.run(m.chat("a", [{"role": "user", "content": "hi"}]))
    assert out["choices"][0]["message"]["content"] == "ok"
    asyncio.run(m.chat("a", [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "ok"}, {"role": "user", "content": "more"}]))
    text = tok.decode(m.get("a").tokens)
    assert text == "[gMASK]<sop><|user|>\nhi<|assistant|>\nok<|user|>\nmore<|assistant|>\nok<|user|>"      # no doubled role tag
    # a diverging request forks a branch; samples come from the leaves only
    asyncio.run(m.chat("a", [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "ok"}, {"role": "user", "content": "other"}]))
    got = session_samples(m, "a", types.SimpleNamespace())
    assert len(got) == 2 and all(isinstance(x, Sample) for x in got)
    a = Sample(tokens=[1, 2, 3, 9], response_length=1)
    b = Sample(tokens=[1, 2, 3, 8], response_length=1)
    c = Sample(tokens=[1, 2, 4, 8], response_length=1)
    assert drop_same_prompt_retries([a, b, c]) == [b, c]
    del s
