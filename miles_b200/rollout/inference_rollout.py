"""Class-based rollout function (default `--rollout-function-path`).

Behaviour (reference: miles/rollout/inference_rollout/inference_rollout_common.py:31-236 and
inference_rollout_train.py:26-193): keep submitting prompt groups (in units of
`over_sampling_batch_size`) until `rollout_batch_size` groups have passed the dynamic-sampling
filter; then abort what is still in flight — with `--partial-rollout` the partial trajectories go
back into the data-source buffer and resume next rollout.  Each sample is generated
token-in-token-out (`input_ids` in, `output_token_logprobs` out; no re-tokenisation) and scored by the
reward hub.
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field
from typing import Any, Callable

from ..types import Sample, Status, decode_routed_experts
from ..utils.misc import load_function
from .rm_hub import async_rm, batched_async_rm


@dataclass
class RolloutFnTrainInput:
    rollout_id: int


@dataclass
class RolloutFnEvalInput:
    rollout_id: int


@dataclass
class RolloutFnTrainOutput:
    samples: list[list[Sample]]
    metrics: dict = field(default_factory=dict)


@dataclass
class RolloutFnEvalOutput:
    data: dict[str, dict[str, Any]]
    metrics: dict = field(default_factory=dict)


@dataclass
class GenerateFnInput:
    args: Any
    sample: Sample
    sampling_params: dict
    client: Any
    evaluation: bool = False


@dataclass
class GenerateFnOutput:
    samples: Sample | list[Sample]


# ---- request payload / response parsing ------------------------------------------------------------

def compute_request_payload(args, input_ids: list[int], sampling_params: dict, *, return_routed_experts: bool = False):
    """Returns (payload | None, status): a non-positive token budget yields TRUNCATED without a call
    (reference: miles/rollout/generate_utils/generate_endpoint_utils.py:57-91)."""
    sp = dict(sampling_params)
    max_ctx = getattr(args, "rollout_max_context_len", None)
    if max_ctx is not None:
        sp["max_new_tokens"] = min(sp["max_new_tokens"], max_ctx - len(input_ids))
    if sp["max_new_tokens"] <= 0:
        return None, Status.TRUNCATED
    payload = {"input_ids": list(input_ids), "sampling_params": sp, "return_logprob": True}
    if return_routed_experts:
        payload["return_routed_experts"] = True
    return payload, None


def update_sample_from_response(args, sample: Sample, payload: dict, output: dict, *, num_layers: int = 0, topk: int = 0,
                                trainable: bool = True):
    meta = output["meta_info"]
    pairs = meta.get("output_token_logprobs") or []
    new_ids = [int(p[1]) for p in pairs]
    new_lps = [float(p[0]) for p in pairs]
    if not sample.tokens:
        sample.tokens = list(payload["input_ids"])
    sample.append_response(new_ids, new_lps, text=output.get("text", ""), trainable=trainable)
    if "routed_experts" in meta and num_layers and topk:
        sample.rollout_routed_experts = decode_routed_experts(meta["routed_experts"], len(sample.tokens), num_layers, topk)
    sample.update_from_meta_info(meta, num_new_tokens=len(new_ids))


async def generate_single_turn(inp: GenerateFnInput) -> GenerateFnOutput:
    args, sample, client = inp.args, inp.sample, inp.client
    if not sample.tokens:
        assert client.tokenizer is not None, "string prompts need a tokenizer"
        sample.tokens = client.tokenizer(sample.prompt, add_special_tokens=False)["input_ids"]
    sp = dict(inp.sampling_params)
    # resume of a partial sample: the budget shrinks by what was already generated
    sp["max_new_tokens"] = sp["max_new_tokens"] - sample.response_length
    want_routing = getattr(args, "use_rollout_routing_replay", False)
    payload, status = compute_request_payload(args, sample.tokens, sp, return_routed_experts=want_routing)
    if payload is None:
        sample.status = status
        return GenerateFnOutput(sample)
    output = await client.generate(payload, routing_key=sample.routing_key)
    update_sample_from_response(args, sample, payload, output, num_layers=client.num_moe_layers, topk=client.moe_topk)
    return GenerateFnOutput(sample)


# ---- one sample / one group ----------------------------------------------------------------------

async def generate_and_rm(args, sample: Sample, sampling_params: dict, client, state, evaluation=False) -> Sample | list[Sample]:
    if sample.status in (Status.COMPLETED, Status.TRUNCATED) and sample.reward is not None:
        return sample
    if state.aborted:
        sample.status = Status.ABORTED
        return sample
    path = sample.generate_function_path or getattr(args, "custom_generate_function_path", None)
    gen_fn = load_function(path) if path else generate_single_turn
    t0 = time.time()
    out = await gen_fn(GenerateFnInput(args, sample, sampling_params, client, evaluation))
    result = out.samples if isinstance(out, GenerateFnOutput) else out
    samples = result if isinstance(result, list) else [result]
    if not getattr(args, "group_rm", False):
        for s in samples:
            if s.status != Status.ABORTED and s.reward is None:
                s.reward = await async_rm(args, s)
    return result


async def generate_and_rm_group(args, group: list[Sample], sampling_params: dict, client, state, evaluation=False):
    if state.aborted:
        return group
    results = await asyncio.gather(*[generate_and_rm(args, s, dict(sampling_params), client, state, evaluation) for s in group])
    flat: list[Sample] = []
    for r in results:
        flat.extend(r if isinstance(r, list) else [r])
    if getattr(args, "group_rm", False) and not state.aborted:
        todo = [s for s in flat if s.status != Status.ABORTED and s.reward is None]
        rewards = await batched_async_rm(args, todo)
        for s, r in zip(todo, rewards):
            s.reward = r
    return flat


class _State:
    def __init__(self):
        self.aborted = False


def check_reward_nonzero_std(args, group: list[Sample], **kw) -> bool:
    """Dynamic-sampling filter (DAPO): keep a group only when its rewards differ."""
    rs = [s.get_reward_value(getattr(args, "reward_key", None)) for s in group]
    return len(set(rs)) > 1


class InferenceRolloutFn:
    """`fn(RolloutFnTrainInput | RolloutFnEvalInput)`; constructed once per run with shared state."""

    def __init__(self, args, data_source, client, eval_sources: dict[str, Any] | None = None):
        self.args, self.data_source, self.client = args, data_source, client
        self.eval_sources = eval_sources or {}
        path = getattr(args, "dynamic_sampling_filter_path", None)
        self.dynamic_filter: Callable | None = load_function(path) if path else None
        path = getattr(args, "rollout_sample_filter_path", None)
        self.sample_filter: Callable | None = load_function(path) if path else None

    def sampling_params(self, evaluation=False) -> dict:
        a = self.args
        sp = {
            "temperature": a.rollout_temperature, "top_p": a.rollout_top_p, "top_k": a.rollout_top_k,
            "max_new_tokens": a.rollout_max_response_len, "stop_token_ids": a.rollout_stop_token_ids or [],
            "skip_special_tokens": a.rollout_skip_special_tokens, "no_stop_trim": True,
        }
        if evaluation:
            if a.eval_temperature is not None:
                sp["temperature"] = a.eval_temperature
            if a.eval_top_p is not None:
                sp["top_p"] = a.eval_top_p
            if a.eval_max_response_len is not None:
                sp["max_new_tokens"] = a.eval_max_response_len
        return sp

    def __call__(self, inp):
        coro = self.eval_async(inp) if isinstance(inp, RolloutFnEvalInput) else self.train_async(inp)
        try:
            asyncio.get_running_loop()
        except RuntimeError:
            return asyncio.run(coro)
        raise RuntimeError("InferenceRolloutFn called from a running loop; await train_async/eval_async instead")

    async def train_async(self, inp: RolloutFnTrainInput) -> RolloutFnTrainOutput:
        args = self.args
        target = args.rollout_batch_size
        over = args.over_sampling_batch_size or target
        state = _State()
        sp = self.sampling_params()
        pending: set[asyncio.Task] = set()
        task_group: dict[asyncio.Task, list[Sample]] = {}
        done_groups: list[list[Sample]] = []
        dropped = 0
        t0 = time.time()
        await self.client.begin()
        while len(done_groups) < target:
            while len(done_groups) + len(pending) < target:
                for g in self.data_source.get_samples(over):
                    t = asyncio.ensure_future(generate_and_rm_group(args, g, sp, self.client, state))
                    task_group[t] = g
                    pending.add(t)
            finished, pending = await asyncio.wait(pending, return_when=asyncio.FIRST_COMPLETED)
            for t in finished:
                group = t.result()
                task_group.pop(t, None)
                if self.dynamic_filter is not None and not self.dynamic_filter(args, group):
                    dropped += 1
                    continue
                if len(done_groups) < target:
                    done_groups.append(group)
        # abort leftovers
        state.aborted = True
        if pending:
            await self.client.abort_all()
            leftovers = await asyncio.gather(*pending)
            if getattr(args, "partial_rollout", False):
                keep = []
                for g in leftovers:
                    for s in g:
                        if s.status == Status.ABORTED:
                            s.status = Status.PENDING
                            s.reward = None
                    if any(s.response_length > 0 for s in g) and len(g) == args.n_samples_per_prompt:
                        keep.append(g)
                if keep:
                    self.data_source.add_samples(keep)
        await self.client.finish()
        done_groups.sort(key=lambda g: g[0].index if g and g[0].index is not None else 0)
        if self.sample_filter is not None:
            self.sample_filter(args, done_groups)
        n_tok = sum(s.response_length for g in done_groups for s in g)
        dt = time.time() - t0
        metrics = {"rollout/dynamic_filter_dropped": dropped, "perf/rollout_time": dt,
                   "perf/rollout_tokens_per_sec": n_tok / max(dt, 1e-9)}
        return RolloutFnTrainOutput(done_groups, metrics)

    async def eval_async(self, inp: RolloutFnEvalInput) -> RolloutFnEvalOutput:
        args = self.args
        state = _State()
        sp = self.sampling_params(evaluation=True)
        await self.client.begin()
        data = {}
        for name, src in self.eval_sources.items():
            n_prompts = len(src) or 1
            saved = args.n_samples_per_prompt
            groups = src.get_samples(n_prompts)
            outs = await asyncio.gather(*[generate_and_rm_group(args, g[: args.n_samples_per_eval_prompt], sp, self.client, state, True)
                                          for g in groups])
            flat = [s for g in outs for s in g]
            key = getattr(args, "eval_reward_key", None) or getattr(args, "reward_key", None)
            data[name] = {"rewards": [s.get_reward_value(key) for s in flat],
                          "truncated": [s.status == Status.TRUNCATED for s in flat], "samples": flat}
        await self.client.finish()
        return RolloutFnEvalOutput(data)


def generate_rollout(args, rollout_id, data_source, evaluation=False, client=None):
    """Function-style legacy entry (reference: miles/rollout/sglang_rollout.py:147-717)."""
    fn = InferenceRolloutFn(args, data_source, client)
    return fn(RolloutFnEvalInput(rollout_id) if evaluation else RolloutFnTrainInput(rollout_id))
