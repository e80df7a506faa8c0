"""Multi-turn / tool-call generation, filters, prompt scoring and on-policy distillation on the CPU engine."""
import asyncio
from types import SimpleNamespace

import torch

from miles_b200.engine.engine import Engine
from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import ForwardMeta
from miles_b200.rollout import filter_hub, generate_hub, opd
from miles_b200.rollout.client import InProcEngineClient
from miles_b200.rollout.inference_rollout import GenerateFnInput
from miles_b200.types import Sample, Status


def _client(seed=0):
    eng = Engine(PRESETS["tiny"], device="cpu", dtype=torch.float32, seed=seed, num_blocks=128, block_size=4)
    return eng, InProcEngineClient([eng])


class CountingEnv:
    """Answers every turn with two fixed observation tokens; done after the third model turn."""

    def __init__(self, args, sample):
        self.turns = 0

    def step(self, text, ids):
        self.turns += 1
        return [7, 8], self.turns >= 3, {"reward": float(self.turns)}


def _args(**kw):
    base = dict(rollout_max_context_len=None, use_rollout_routing_replay=False, multi_turn_env_path=None, max_turns=8,
                tools_path=None, reward_key=None, rollout_max_response_len=64)
    base.update(kw)
    return SimpleNamespace(**base)


def test_multi_turn_masks_observations_and_keeps_exact_tokens():
    eng, client = _client()
    args = _args(multi_turn_env_path="tests.test_generate_hub.CountingEnv")
    s = Sample(tokens=[5, 6, 7, 9])
    sp = {"temperature": 0.0, "max_new_tokens": 40}

    args.max_tokens_per_turn = 4

    async def go():
        await client.begin()
        out = await generate_hub.generate_multi_turn(GenerateFnInput(args, s, sp, client))
        await client.finish()
        return out.samples

    r = asyncio.run(go())
    assert r.status == Status.COMPLETED and r.reward == 3.0
    # 3 model turns of 4 tokens with 2 observation tokens after the first two
    assert r.response_length == 4 + 2 + 4 + 2 + 4
    assert r.loss_mask == [1] * 4 + [0] * 2 + [1] * 4 + [0] * 2 + [1] * 4
    assert r.tokens[4 + 4: 4 + 6] == [7, 8]
    # the trajectory is what the model saw: greedy re-decode of each model turn from the accumulated ids agrees
    T = len(r.tokens)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    lp = torch.log_softmax(eng.model.logits(eng.model(torch.tensor(r.tokens, dtype=torch.int32), meta)).float(), -1)
    P = 4
    for j, (tok, m, got) in enumerate(zip(r.tokens[P:], r.loss_mask, r.rollout_log_probs)):
        if m:
            assert int(lp[P + j - 1].argmax()) == tok
            assert abs(float(lp[P + j - 1, tok]) - got) < 1e-4


def test_tool_call_parsing_and_env():
    text = 'let me check <tool_call>{"name": "add", "arguments": {"a": 2, "b": 3}}</tool_call> and <tool_call>{bad}</tool_call>'
    assert generate_hub.parse_tool_calls(text) == [{"name": "add", "arguments": {"a": 2, "b": 3}}]
    s = Sample(tokens=[1])
    env = generate_hub.ToolEnv(_args(), s, tools={"add": lambda a, b: a + b, "boom": lambda: 1 / 0})
    obs, done, _ = asyncio.run(env.step(text, []))
    assert not done and "<tool_response>\n5\n</tool_response>" in obs
    obs, done, _ = asyncio.run(env.step('<tool_call>{"name": "boom", "arguments": {}}</tool_call>', []))
    assert "ZeroDivisionError" in obs
    obs, done, _ = asyncio.run(env.step('<tool_call>{"name": "nope", "arguments": {}}</tool_call>', []))
    assert "unknown tool" in obs
    _, done, _ = asyncio.run(env.step("final answer: 5", []))
    assert done and len(s.metadata["tool_calls"]) == 3


def test_filters():
    args = _args()
    mk = lambda r, st=Status.COMPLETED, n=3: Sample(tokens=[1] * (1 + n), response_length=n, reward=r, status=st)
    assert filter_hub.check_reward_nonzero_std(args, [mk(0.0), mk(1.0)])
    assert not filter_hub.check_reward_nonzero_std(args, [mk(1.0), mk(1.0)])
    assert not filter_hub.check_no_truncated(args, [mk(1.0), mk(0.0, Status.TRUNCATED)])
    groups = [[mk(1.0), mk(0.0, Status.TRUNCATED)]]
    filter_hub.remove_truncated(args, groups)
    assert [s.remove_sample for s in groups[0]] == [False, True]
    buf = [[mk(0, n=2)], [mk(0, n=9)], [mk(0, n=5)]]
    got = filter_hub.pop_longest_first(args, 0, buf, 2)
    assert [g[0].response_length for g in got] == [9, 5] and len(buf) == 1


def test_prompt_logprobs_and_opd_scoring():
    eng, client = _client(seed=0)
    teacher_eng, teacher = _client(seed=1)
    s = Sample(tokens=[5, 6, 7, 9])

    async def go():
        await client.begin()
        out = await client.generate({"input_ids": s.tokens, "sampling_params": {"temperature": 1.0, "max_new_tokens": 6, "seed": 3},
                                     "return_logprob": True})
        await client.finish()
        pairs = out["meta_info"]["output_token_logprobs"]
        s.append_response([p[1] for p in pairs], [p[0] for p in pairs])
        args = _args(opd_teacher_client=teacher, opd_task_rm_type=None)
        await teacher.begin()
        r = await opd.opd_reward(args, s)
        await teacher.finish()
        return r

    assert asyncio.run(go()) == 0.0
    assert len(s.teacher_log_probs) == 6 and len(s.opd_reverse_kl) == 6
    # teacher log-probs equal a plain forward of the teacher model over the whole sequence
    T = len(s.tokens)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    lp = torch.log_softmax(teacher_eng.model.logits(teacher_eng.model(torch.tensor(s.tokens, dtype=torch.int32), meta)).float(), -1)
    want = [float(lp[4 + j - 1, t]) for j, t in enumerate(s.tokens[4:])]
    assert max(abs(a - b) for a, b in zip(want, s.teacher_log_probs)) < 1e-4
    # scoring from position 0 returns None for the first token
    out = teacher_eng.generate(s.tokens, {"temperature": 0.0, "max_new_tokens": 1})
    assert "input_token_logprobs" not in out["meta_info"]
    req = teacher_eng.add_request(s.tokens, {"temperature": 0.0, "max_new_tokens": 1}, logprob_start_len=0)
    while not req.done.is_set():
        teacher_eng.step()
    itl = req.to_response(teacher_eng)["meta_info"]["input_token_logprobs"]
    assert len(itl) == T and itl[0][0] is None and abs(itl[5][0] - want[1]) < 1e-4
    assert opd.topk_reverse_kl([[-0.1, -3.0]], [[-0.1, -3.0]])[0] < 1e-9


def test_opd_teacher_fleet_topk_strategies_and_trainer_side_teacher(tmp_path):
    import pytest

    # teacher fleet: routing by the sample's metadata key, default fallback, malformed entries
    assert opd.parse_teacher_urls(["math=http://h1:1/generate", "http://h3:3"]) == {"math": "http://h1:1/generate", "default": "http://h3:3"}
    with pytest.raises(ValueError):
        opd.parse_teacher_urls(["a=http://x", "a=http://y"])
    e1, t1 = _client(seed=1)
    e2, t2 = _client(seed=2)
    s_math = Sample(tokens=[5, 6, 7, 9], metadata={"opd_teacher": "math"})
    s_other = Sample(tokens=[5, 6, 7, 9], metadata={"opd_teacher": "poetry"})
    for s in (s_math, s_other):
        s.append_response([3, 4, 5], [-1.0, -1.0, -1.0])

    async def go(k=0, strategy="only-teacher"):
        args = _args(opd_teacher_client={"math": t1, "default": t2}, opd_teacher_key="opd_teacher", opd_task_rm_type=None,
                     opd_log_prob_top_k=k, opd_top_k_strategy=strategy, opd_reward_weight_mode="student_p")
        for t in (t1, t2):
            await t.begin()
        for s in (s_math, s_other):
            await opd.opd_reward(args, s)
        for t in (t1, t2):
            await t.finish()

    asyncio.run(go())
    assert s_math.teacher_log_probs != s_other.teacher_log_probs                   # two different teachers answered
    # top-k scoring: the teacher's k most likely tokens per response position, sorted, log-probs of a distribution
    asyncio.run(go(k=4))
    req = e1.add_request(s_math.tokens, {"temperature": 0.0, "max_new_tokens": 1}, logprob_start_len=4, top_logprobs_num=4)
    while not req.done.is_set():
        e1.step()
    meta = req.to_response(e1)["meta_info"]
    tops = meta["input_top_logprobs"]
    assert len(tops) == 3 and all(len(row) == 4 and row[0][0] >= row[-1][0] for row in tops)
    assert all(abs(tops[j][0][0]) < 20 and meta["input_token_logprobs"][j][0] <= tops[j][0][0] + 1e-6 for j in range(3))
    assert len(s_math.opd_reverse_kl) == 3                                          # only-teacher: computed without student lists
    # strategies on a hand-made position
    st, te = {1: -0.2, 2: -2.0}, {1: -0.5, 3: -1.0}
    assert opd.set_reverse_kl(st, te, "intersection") == pytest.approx(0.0)          # one shared token: both renormalise to 1
    assert opd.set_reverse_kl(st, te, "only-student") > 0 and opd.set_reverse_kl(st, te, "union", "teacher_p") != 0
    assert opd.set_reverse_kl(st, te, "xor", "none") == pytest.approx(((-2.0 - -1.0) + (-2.0 - -1.0)) / 2)
    with pytest.raises(ValueError):
        opd.set_reverse_kl(st, te, "nearest")
    # --opd-type megatron: the trainer scores with a second set of weights loaded from a checkpoint
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_e2e import BASE, _run
    from miles_b200.args import parse_args

    ck = str(tmp_path / "teacher")
    _run(f"--num-rollout 1 --save {ck} --save-interval 1 --seed 77")
    with pytest.raises(ValueError):
        parse_args((BASE + " --use-opd").split())
    h = _run(f"--use-opd --opd-type megatron --opd-teacher-load {ck} --opd-teacher-ckpt-step 0 --opd-kl-coef 0.5 --num-rollout 1")
    assert "perf/teacher_log_probs_time" in h.rows[0] and h.series("train/grad_norm")[0] > 0
