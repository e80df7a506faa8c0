"""Generate functions beyond single-turn: multi-turn with an environment, and agentic tool calling.

Select with `--custom-generate-function-path miles_b200.rollout.generate_hub.generate_multi_turn` (or
`…generate_with_tools`).  Counterparts of the reference's generate hub (miles/rollout/generate_hub/multi_turn.py,
agentic_tool_call.py): every turn is token-in-token-out — the exact ids the engine produced are appended to the
trajectory with `loss_mask = 1`, environment / tool output is tokenised once, appended with `loss_mask = 0`, and the
next request continues from the accumulated ids, so the trainer sees precisely the sequence the engine saw.

Environment protocol (`--multi-turn-env-path module.Class`): `env = Class(args, sample)`;
`obs, done, info = await env.step(response_text, response_ids)` — `obs` is text (needs a tokenizer) or a list of ids;
`info` may carry `reward`.
"""
from __future__ import annotations

import asyncio
import json
import re
from typing import Any, Callable

from ..types import Sample, Status
from ..utils.misc import load_function
from .inference_rollout import GenerateFnInput, GenerateFnOutput, compute_request_payload, update_sample_from_response


def _encode(client, obs) -> list[int]:
    if isinstance(obs, str):
        assert client.tokenizer is not None, "text observations need a tokenizer"
        return client.tokenizer(obs, add_special_tokens=False)["input_ids"]
    return [int(t) for t in obs]


async def _one_turn(inp: GenerateFnInput, sample: Sample, budget: int) -> tuple[str, list[int]] | None:
    """One engine call continuing `sample.tokens`; returns (text, new ids) or None when no budget is left."""
    args, client = inp.args, inp.client
    sp = dict(inp.sampling_params)
    sp["max_new_tokens"] = min(sp["max_new_tokens"], budget)
    payload, status = compute_request_payload(args, sample.tokens, sp,
                                              return_routed_experts=getattr(args, "use_rollout_routing_replay", False))
    if payload is None:
        sample.status = status
        return None
    before = len(sample.tokens)
    out = await client.generate(payload, routing_key=sample.routing_key)
    update_sample_from_response(args, sample, payload, out, num_layers=client.num_moe_layers, topk=client.moe_topk)
    return out.get("text", ""), sample.tokens[before:]


async def generate_multi_turn(inp: GenerateFnInput) -> GenerateFnOutput:
    args, sample, client = inp.args, inp.sample, inp.client
    if not sample.tokens:
        assert client.tokenizer is not None, "string prompts need a tokenizer"
        sample.tokens = client.tokenizer(sample.prompt, add_special_tokens=False)["input_ids"]
    env_path = getattr(args, "multi_turn_env_path", None) or (sample.metadata or {}).get("env_path")
    assert env_path, "--multi-turn-env-path (or sample.metadata['env_path']) names the environment class"
    env = load_function(env_path)(args, sample)
    max_turns = getattr(args, "max_turns", 8)
    total_budget = inp.sampling_params["max_new_tokens"]
    per_turn = getattr(args, "max_tokens_per_turn", None) or total_budget
    for _turn in range(max_turns):
        left = total_budget - sample.response_length
        got = await _one_turn(inp, sample, min(left, per_turn))
        if got is None or sample.status == Status.ABORTED:
            break
        if sample.status == Status.TRUNCATED and sample.response_length >= total_budget:
            break                                   # the whole trajectory ran out of budget, not just this turn
        text, ids = got
        res = env.step(text, ids)
        obs, done, info = await res if asyncio.iscoroutine(res) else res
        if info and "reward" in info:
            sample.reward = info["reward"]
        if done:
            sample.status = Status.COMPLETED
            break
        obs_ids = _encode(client, obs)
        if sample.response_length + len(obs_ids) >= total_budget:
            sample.status = Status.TRUNCATED
            break
        sample.append_response(obs_ids, None, text=obs if isinstance(obs, str) else "", trainable=False)
    else:
        sample.status = Status.TRUNCATED
    return GenerateFnOutput(sample)


# ---- tool calling ----------------------------------------------------------------------------------------

TOOL_CALL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str) -> list[dict]:
    """Qwen/Hermes-style `<tool_call>{"name": …, "arguments": {…}}</tool_call>` blocks."""
    calls = []
    for m in TOOL_CALL_RE.finditer(text):
        try:
            d = json.loads(m.group(1))
            if isinstance(d, dict) and "name" in d:
                calls.append({"name": d["name"], "arguments": d.get("arguments", {})})
        except json.JSONDecodeError:
            continue
    return calls


def format_tool_response(results: list[Any]) -> str:
    return "".join(f"\n<tool_response>\n{r if isinstance(r, str) else json.dumps(r)}\n</tool_response>" for r in results) + "\n"


class ToolEnv:
    """Environment that executes tool calls found in the model's turn.  `tools`: name → callable(**arguments) (sync or
    async).  The episode ends at the first turn without a tool call."""

    def __init__(self, args, sample: Sample, tools: dict[str, Callable] | None = None):
        self.args, self.sample = args, sample
        if tools is None:
            path = getattr(args, "tools_path", None) or (sample.metadata or {}).get("tools_path")
            tools = load_function(path) if path else {}
            if callable(tools):
                tools = tools(args, sample)
        self.tools = tools
        self.calls: list[dict] = []

    async def step(self, text: str, ids: list[int]):
        calls = parse_tool_calls(text)
        if not calls:
            return "", True, {}
        results = []
        for c in calls:
            fn = self.tools.get(c["name"])
            if fn is None:
                results.append({"error": f"unknown tool {c['name']}"})
                continue
            try:
                r = fn(**c["arguments"]) if isinstance(c["arguments"], dict) else fn(c["arguments"])
                results.append(await r if asyncio.iscoroutine(r) else r)
            except Exception as e:   # a failing tool is an observation, not a crash of the rollout
                results.append({"error": f"{type(e).__name__}: {e}"})
        self.calls.extend(calls)
        self.sample.metadata.setdefault("tool_calls", []).extend(calls)
        return format_tool_response(results), False, {}


async def generate_with_tools(inp: GenerateFnInput) -> GenerateFnOutput:
    """Agentic tool-call loop: `generate_multi_turn` with `ToolEnv` (tools from `--tools-path module.dict_or_factory`)."""
    args = inp.args
    if not getattr(args, "multi_turn_env_path", None):
        import copy

        args = copy.copy(args)
        args.multi_turn_env_path = "miles_b200.rollout.generate_hub.ToolEnv"
        inp = GenerateFnInput(args, inp.sample, inp.sampling_params, inp.client, inp.evaluation)
    return await generate_multi_turn(inp)
