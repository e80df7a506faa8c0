"""Reward hub, data source, argument validation and the native runtime (CPU)."""
import asyncio
import json
from types import SimpleNamespace

import pytest

from miles_b200.rollout import rm_hub
from miles_b200.types import RewardSpec, Sample


def _s(response, label=None, **kw):
    return Sample(prompt="q", response=response, label=label, **kw)


def _rm(rm_type, sample, **kw):
    args = SimpleNamespace(rm_type=rm_type, custom_rm_path=None, **kw)
    return asyncio.run(rm_hub.async_rm(args, sample))


def test_math_graders():
    assert rm_hub.last_boxed(r"so \boxed{\frac{1}{2}} and finally \boxed{42}") == "42"
    assert rm_hub.last_boxed(r"\boxed{a{b}c}") == "a{b}c"
    assert rm_hub.math_equal("0.5", "1/2") or rm_hub.math_equal(r"\frac{1}{2}", "1/2")
    assert _rm("math", _s(r"The answer is \boxed{42}.", "42")) == 1.0
    assert _rm("math", _s(r"The answer is \boxed{41}.", "42")) == 0.0
    assert _rm("boxed_math", _s(r"\boxed{ 3 }", "3")) == 1.0
    d = _rm("dapo", _s("Answer: 7", "7"))
    assert isinstance(d, dict) and "score" in d
    assert _rm("deepscaler", _s(r"<think>hm</think> \boxed{5}", "5")) == 1.0


def test_text_graders():
    assert _rm("f1", _s("the cat sat", "the cat sat")) == pytest.approx(1.0)
    assert 0 < _rm("f1", _s("the cat", "the cat sat down")) < 1
    assert _rm("gpqa", _s("I think the answer is (B).", "B")) == 1.0
    assert _rm("gpqa", _s("Answer: C", "B")) == 0.0
    assert _rm("deterministic_random", _s("x", tokens=[1, 2, 3])) == _rm("deterministic_random", _s("x", tokens=[1, 2, 3]))


def test_reward_spec_overrides_args_and_custom_path():
    s = _s(r"\boxed{1}", "1", reward_spec=RewardSpec(rm_type="math"))
    assert _rm("f1", s) == 1.0
    args = SimpleNamespace(rm_type=None, custom_rm_path="tests.test_rollout._custom_rm")
    assert asyncio.run(rm_hub.async_rm(args, _s("abc"))) == 3.0
    with pytest.raises(ValueError):
        asyncio.run(rm_hub.async_rm(SimpleNamespace(rm_type=None, custom_rm_path=None), _s("abc")))


def _custom_rm(args, sample, **kw):
    return float(len(sample.response))


def test_data_source_epochs_state_and_buffer(tmp_path):
    from miles_b200.rollout.data_source import RolloutDataSourceWithBuffer

    p = tmp_path / "prompts.jsonl"
    with open(p, "w") as f:
        for i in range(5):
            f.write(json.dumps({"input": f"q{i}", "label": str(i)}) + "\n")
    from miles_b200.args import parse_args

    args = parse_args(f"--model-name tiny --num-rollout 1 --prompt-data {p} --input-key input --label-key label "
                      f"--n-samples-per-prompt 2 --rollout-batch-size 2 --save {tmp_path} --load {tmp_path}".split())
    ds = RolloutDataSourceWithBuffer(args, None)
    assert len(ds) == 5
    g = ds.get_samples(3)
    assert [x[0].label for x in g] == ["0", "1", "2"] and all(len(x) == 2 for x in g)
    assert g[0][0].index == 0 and g[0][1].index == 1 and g[1][0].group_index == 1
    ds.save(0)
    g2 = ds.get_samples(3)                                      # wraps into the next epoch
    assert [x[0].label for x in g2] == ["3", "4", "0"]
    ds.add_samples([g2[2]])                                     # aborted group goes back to the buffer
    assert ds.buffer_length() == 1
    assert ds.get_samples(1)[0][0].label == "0"
    fresh = RolloutDataSourceWithBuffer(args, None)
    fresh.load(0)
    assert [x[0].label for x in fresh.get_samples(2)] == ["3", "4"]


def test_args_validation():
    from miles_b200.args import parse_args

    a = parse_args("--model-name tiny --rollout-batch-size 8 --n-samples-per-prompt 4 --num-rollout 1 --rm-type math".split())
    assert a.global_batch_size == 32 and a.num_steps_per_rollout == 1
    a = parse_args("--model-name tiny --rollout-batch-size 8 --n-samples-per-prompt 4 --global-batch-size 16 --num-rollout 1".split())
    assert a.num_steps_per_rollout == 2
    with pytest.raises((AssertionError, SystemExit)):
        parse_args("--model-name tiny --rollout-batch-size 8 --n-samples-per-prompt 4 --global-batch-size 12 --num-rollout 1".split())
    a = parse_args("--model-name tiny --num-rollout 1 --sglang-mem-fraction-static 0.5 --sglang-enable-ep-moe".split())
    assert a.engine_kwargs["mem_fraction_static"] == 0.5 and a.engine_kwargs["enable_ep_moe"] is True


def test_native_runtime_allocator_and_router_core():
    from miles_b200.native import runtime as rt

    if not rt.available():
        rt.build()
    assert rt.available()
    al = rt.NativeBlockAllocator(16)
    a = al.alloc(5)
    assert len(a) == 5 and al.num_free == 11 and al.alloc(12) is None
    al.share(a)
    al.release(a)
    assert al.num_free == 11
    al.release(a)
    assert al.num_free == 16
    core = rt.NativeRouterCore(0)
    w = [core.add_worker() for _ in range(3)]
    picks = [core.pick("least_active") for _ in range(6)]
    assert sorted(picks) == [0, 0, 1, 1, 2, 2]
    core.set_health(w[1], False)
    assert 1 not in {core.pick("round_robin") for _ in range(6)}
    k = core.pick("consistent_hashing", "session-a")
    assert all(core.pick("consistent_hashing", "session-a") == k for _ in range(4))


def test_sft_rollout_masks_assistant_turns_only(tmp_path):
    """Multi-turn conversations → token ids + a loss mask that is 1 exactly on what the assistant produced (content and
    end-of-turn token), for a ChatML-style family and for one that ends turns with the next role tag."""
    import json
    from types import SimpleNamespace

    from miles_b200.rollout.inference_rollout import RolloutFnTrainInput
    from miles_b200.rollout.sft_rollout import SftRolloutFn, conversation_tokens_and_mask
    from miles_b200.session.tito import ByteChatTokenizer, TitoTokenizer
    from miles_b200.types import Sample

    tok = ByteChatTokenizer()
    tito = TitoTokenizer(tok, "qwen3")
    msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": "q1"}, {"role": "assistant", "content": "a1"},
            {"role": "tool", "content": "t"}, {"role": "assistant", "content": "a2"}]
    ids, mask = conversation_tokens_and_mask(tito, msgs)
    assert ids == tito.encode(tito.render(msgs))                              # the pieces add up to the rendered conversation
    trained = tok.decode([t for t, m in zip(ids, mask) if m])
    assert trained == "a1<|im_end|>a2<|im_end|>"
    glm = TitoTokenizer(ByteChatTokenizer(["[gMASK]", "<sop>", "<|system|>", "<|user|>", "<|assistant|>", "<|observation|>"]), "glm47")
    ids2, mask2 = conversation_tokens_and_mask(glm, msgs[1:3])
    assert glm.tok.decode([t for t, m in zip(ids2, mask2) if m]) == "a1<|user|>"       # the turn ends by emitting the next role tag

    class Source:
        tokenizer = tok

        def get_samples(self, n):
            return [[Sample(prompt=msgs)], [Sample(prompt="what?", label="that")], [Sample(prompt=[{"role": "user", "content": "no answer"}])]][:n]

    fn = SftRolloutFn(SimpleNamespace(rollout_batch_size=3, tito_model="qwen3", rollout_max_context_len=None), Source())
    out = fn(RolloutFnTrainInput(0))
    assert len(out.samples) == 2 and out.metrics["rollout/sft_dropped"] == 1.0   # a conversation without an assistant turn trains nothing
    s = out.samples[0][0]
    assert len(s.loss_mask) == s.response_length and s.loss_mask[0] == 1 and sum(s.loss_mask) == len(tok("a1<|im_end|>a2<|im_end|>")["input_ids"])
    s2 = out.samples[1][0]
    assert tok.decode(s2.tokens[-s2.response_length:]).startswith("that<|im_end|>")
    del json


def test_recipes_build_commands_that_parse():
    """Every launch recipe yields an argument list the trainer's parser accepts; run.py prints the torchrun command."""
    import io
    import os
    import sys
    from contextlib import redirect_stdout

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import run
    from miles_b200 import recipes
    from miles_b200.args import parse_args

    for name in recipes.RECIPES:
        for mode in ("normal", "debug_minimal", "debug_one_sample"):
            r = recipes.build(name, recipes.Knobs(num_gpus=8, mode=mode, dynamic_sampling=True, use_kl_loss=True))
            a = parse_args(r.args)
            assert a.rollout_batch_size >= 1 and os.path.exists(os.path.join(os.path.dirname(run.__file__), r.entry)), name
    a = parse_args(recipes.build("qwen3-30b-a3b", recipes.Knobs(num_gpus=8, mxfp8=True)).args)
    assert a.expert_model_parallel_size == 8 and a.fp8_recipe == "mxfp8" and a.max_tokens_per_gpu == 32768 and a.use_rollout_routing_replay
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert run.main(["qwen3-4b", "--num-gpus", "4", "--mode", "debug_minimal", "--dry-run", "--", "--lr", "3e-6"]) == 0
    cmd = buf.getvalue()
    assert "--nproc-per-node=4" in cmd and "train.py" in cmd and cmd.rstrip().endswith("--lr 3e-6")
    with redirect_stdout(io.StringIO()) as b2:
        run.main(["list"])
    assert "qwen3-235b-a22b" in b2.getvalue()


# ---- balanced local exchange ---------------------------------------------------------------------------------------

def test_plan_group_moves_narrows_the_spread_and_is_deterministic():
    import random

    from miles_b200.orchestration.rollout_executor import plan_group_moves

    rng = random.Random(3)
    for _ in range(20):
        sizes = [[rng.randint(4000, 22000) for _ in range(8)] for _ in range(8)]
        moves = plan_group_moves(sizes)
        assert moves == plan_group_moves([list(s) for s in sizes])
        loads = [sum(s) for s in sizes]
        before = max(loads) - min(loads)
        seen = set()
        for src, i, dst in moves:
            assert (src, i) not in seen and src != dst           # a group moves at most once
            seen.add((src, i))
            loads[src] -= sizes[src][i]
            loads[dst] += sizes[src][i]
        assert sum(loads) == sum(map(sum, sizes))
        assert max(loads) - min(loads) <= before
        assert max(loads) / (sum(loads) / 8) < 1.06               # from ≈ 1.15 for such draws
    assert plan_group_moves([[10, 10], [10, 10]]) == [] and plan_group_moves([[5]]) == []


def _rebalance_body(rank, world):
    import numpy as np

    from miles_b200.orchestration.rollout_executor import RolloutExecutor
    from miles_b200.types import Sample

    def group(gid, n_tok):
        out = []
        for j in range(2):
            s = Sample(index=gid * 2 + j, prompt="p", tokens=list(range(gid, gid + n_tok)), response_length=n_tok // 2,
                       reward=float(gid), loss_mask=[1] * (n_tok // 2), rollout_log_probs=[-0.5] * (n_tok // 2))
            s.rollout_routed_experts = np.full((n_tok - 1, 2, 2), gid, dtype=np.int32)
            out.append(s)
        return out

    mine = [group(10 * rank + i, n) for i, n in enumerate([400, 300, 200, 50] if rank == 0 else [60, 40, 30, 20])]
    ex = RolloutExecutor.__new__(RolloutExecutor)
    ex.gather_group = None
    got = ex._rebalance(mine)
    stride = 1 << 40
    assert len({s.index for g in got for s in g}) == sum(len(g) for g in got)      # ids stay unique on the receiving rank
    assert all((s.index >= stride) == (s.tokens[0] // 10 != rank) for g in got for s in g)
    for g in got:
        for s in g:
            s.index %= stride
    ids = sorted(g[0].index // 2 for g in got)
    tokens = sum(len(s.tokens) for g in got for s in g)
    assert abs(tokens - 1100) <= 100, tokens                                       # 2200 tokens in all, 1900 of them started on rank 0
    for g in got:
        gid = g[0].index // 2
        assert len(g) == 2 and g[0].tokens[0] == gid and g[1].reward == float(gid)
        assert (np.asarray(g[0].rollout_routed_experts) == gid).all() and g[0].rollout_routed_experts.shape[1:] == (2, 2)
    import torch.distributed as dist

    everything: list = [None] * world
    dist.all_gather_object(everything, ids)
    assert sorted(sum(everything, [])) == [0, 1, 2, 3, 10, 11, 12, 13]             # nothing lost, nothing doubled
    if rank == 1:
        assert any(i < 10 for i in ids)                                            # rank 1 received a group of rank 0


def test_balanced_exchange_moves_whole_groups_between_ranks():
    import os
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_distributed

    run_distributed(_rebalance_body, 2, (), timeout=300)
