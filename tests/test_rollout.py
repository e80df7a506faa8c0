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
