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
