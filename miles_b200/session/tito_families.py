"""Chat formats of the model families the token-in-token-out tokenizer knows, and what differs between them at a turn
boundary.

Extending a token trajectory by new messages needs three things per family (reference:
miles/utils/chat_template_utils/tito_tokenizer.py:99-1247 — one class per family with a fixed template, boundary fix-ups in
`merge_tokens`, allowed append roles and the engine-side parser names):

1. a RENDERER of a message list that is prefix-stable (appending a message never rewrites earlier text).  Family templates
   shipped with checkpoints are often not: they strip the reasoning of earlier assistant turns, or fold tool results into
   the previous user turn.  Each family therefore has a fixed renderer here, written from the public chat format;
2. the BOUNDARY rule: which ids the engine's own output leaves out or duplicates at the end of its turn.  Qwen stops at
   `<|im_end|>` but the format continues with a newline; GLM ends a turn by emitting the NEXT role tag (`<|user|>` /
   `<|observation|>`), which must not be rendered a second time; DeepSeek, Llama-3, Gemma and Kimi end with one closing
   token the model usually emits itself;
3. which roles may be appended after an assistant turn, and the names of the reasoning / tool-call parsers the serving
   engine should be started with for this family.

Appended text is rendered against a DUMMY two-message prefix rather than the real history, so the cost of a turn does not
grow with the conversation and nothing in the history can leak into the suffix.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Callable


@dataclass(frozen=True)
class Family:
    name: str
    bos: str = ""                                        # emitted once at the very start
    open: Callable[[str], str] = lambda role: ""         # text that opens a message of `role`
    close: str = ""                                      # text that closes every message
    eot: str = ""                                        # the closing token the model itself samples to end its turn
    after_eot: str = ""                                  # format text after `eot` that the model does not sample
    generation_prompt: str = ""
    think_open: str = "<think>\n"
    think_close: str = "</think>\n\n"
    stop_role_tags: tuple = ()                           # GLM-style: role tags that END the assistant turn when sampled
    tool_role: str = "tool"
    wrap_tool: Callable[[str], str] = lambda c: c
    tool_call: Callable[[dict], str] = lambda call: json.dumps(call, ensure_ascii=False)
    tools_preamble: Callable[[list], str] | None = None  # how tool schemas enter the system prompt
    default_system: str | None = None
    allowed_append_roles: tuple = ("user", "tool", "system")
    reasoning_parser: str | None = None
    tool_call_parser: str | None = None
    extra: dict = field(default_factory=dict)

    # ---- rendering -------------------------------------------------------------------------------------------
    def message(self, m: dict, *, last_assistant: bool = True, keep_reasoning: bool = True) -> str:
        role, content = m["role"], _text(m.get("content"))
        if role == "assistant":
            body = ""
            reasoning = m.get("reasoning_content")
            if reasoning and keep_reasoning:
                body += f"{self.think_open}{reasoning.strip()}{self.think_close.rstrip() if not content else self.think_close}"
            body += content
            for call in m.get("tool_calls") or []:
                fn = call.get("function", call)
                args = fn.get("arguments")
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except ValueError:
                        pass
                body += self.tool_call({"name": fn.get("name"), "arguments": args})
            return self.open("assistant") + body + (self.close or (self.eot if self.extra.get("assistant_closes_with_eot") else ""))
        if role == "tool":
            return self.open(self.tool_role) + self.wrap_tool(content) + self.close
        return self.open(role) + content + self.close

    def render(self, messages: list[dict], add_generation_prompt: bool = False, tools: list | None = None,
               enable_thinking: bool | None = None) -> str:
        msgs = list(messages)
        out = [self.bos]
        sys_extra = self.tools_preamble(tools) if (tools and self.tools_preamble) else ""
        if msgs and msgs[0]["role"] == "system":
            out.append(self.open("system") + _text(msgs[0].get("content")) + sys_extra + self.close)
            msgs = msgs[1:]
        elif sys_extra or self.default_system:
            out.append(self.open("system") + (self.default_system or "") + sys_extra + self.close)
        i = 0
        while i < len(msgs):
            m = msgs[i]
            if m["role"] == "tool" and self.extra.get("group_tool_results"):
                # consecutive tool results share one enclosing turn (Qwen: one user turn with several <tool_response> blocks)
                j = i
                parts = []
                while j < len(msgs) and msgs[j]["role"] == "tool":
                    parts.append(self.wrap_tool(_text(msgs[j].get("content"))))
                    j += 1
                out.append(self.open(self.tool_role) + "\n".join(parts) + self.close)
                i = j
                continue
            out.append(self.message(m))
            i += 1
        if add_generation_prompt:
            out.append(self.generation_prompt)
            if enable_thinking is False and self.extra.get("no_think_prompt"):
                out.append(self.extra["no_think_prompt"])
        return "".join(out)


def _text(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")


# ---- the families ---------------------------------------------------------------------------------------------------

def _qwen_tools(tools: list) -> str:
    lines = "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
    return ("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\nYou are provided with function "
            f"signatures within <tools></tools> XML tags:\n<tools>\n{lines}\n</tools>\n\nFor each function call, return a json object with "
            "function name and arguments within <tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, "
            "\"arguments\": <args-json-object>}\n</tool_call>")


def _qwen_call(call: dict) -> str:
    return "\n<tool_call>\n" + json.dumps(call, ensure_ascii=False) + "\n</tool_call>"


QWEN3 = Family(
    name="qwen3", open=lambda r: f"<|im_start|>{r}\n", close="<|im_end|>\n", eot="<|im_end|>", after_eot="\n",
    generation_prompt="<|im_start|>assistant\n", tool_role="user",
    wrap_tool=lambda c: f"<tool_response>\n{c}\n</tool_response>", tool_call=_qwen_call, tools_preamble=_qwen_tools,
    reasoning_parser="qwen3", tool_call_parser="qwen25",
    extra={"group_tool_results": True, "no_think_prompt": "<think>\n\n</think>\n\n"})

QWEN35 = Family(**{**QWEN3.__dict__, "name": "qwen35", "tool_call_parser": "qwen3_coder",
                   "tool_call": lambda call: ("\n<tool_call>\n<function=" + str(call.get("name")) + ">\n" + "".join(
                       f"<parameter={k}>\n{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}\n</parameter>\n"
                       for k, v in (call.get("arguments") or {}).items()) + "</function>\n</tool_call>")})

QWEN_NEXT = Family(**{**QWEN3.__dict__, "name": "qwen_next", "generation_prompt": "<|im_start|>assistant\n<think>\n",
                      "extra": {"group_tool_results": True}})

GLM47 = Family(
    name="glm47", bos="[gMASK]<sop>", open=lambda r: {"system": "<|system|>\n", "user": "<|user|>\n", "assistant": "<|assistant|>\n",
                                                        "observation": "<|observation|>\n"}[r],
    close="", eot="", generation_prompt="<|assistant|>\n", tool_role="observation", think_open="<think>", think_close="</think>\n",
    stop_role_tags=("<|user|>", "<|observation|>"),
    tool_call=lambda call: "\n<tool_call>" + str(call.get("name")) + "\n" + "".join(
        f"<arg_key>{k}</arg_key>\n<arg_value>{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</arg_value>\n"
        for k, v in (call.get("arguments") or {}).items()) + "</tool_call>",
    reasoning_parser="glm45", tool_call_parser="glm47", extra={"no_think_prompt": "<think></think>\n"})

DEEPSEEK = Family(
    name="deepseek", bos="<｜begin▁of▁sentence｜>",
    open=lambda r: {"system": "", "user": "<｜User｜>", "assistant": "<｜Assistant｜>", "tool": "<｜tool▁output▁begin｜>"}[r],
    close="", eot="<｜end▁of▁sentence｜>", generation_prompt="<｜Assistant｜>", think_open="<think>\n", think_close="\n</think>\n\n",
    wrap_tool=lambda c: c + "<｜tool▁output▁end｜>",
    tool_call=lambda call: ("<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>" + str(call.get("name")) + "\n```json\n"
                            + json.dumps(call.get("arguments"), ensure_ascii=False) + "\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>"),
    reasoning_parser="deepseek-r1", tool_call_parser="deepseekv3", extra={"assistant_closes_with_eot": True})

KIMI = Family(
    name="kimi", open=lambda r: {"system": "<|im_system|>system<|im_middle|>", "user": "<|im_user|>user<|im_middle|>",
                                 "assistant": "<|im_assistant|>assistant<|im_middle|>", "tool": "<|im_system|>tool<|im_middle|>"}[r],
    close="<|im_end|>", eot="<|im_end|>", generation_prompt="<|im_assistant|>assistant<|im_middle|>", think_open="<think>",
    think_close="</think>",
    tool_call=lambda call: ("<|tool_calls_section_begin|><|tool_call_begin|>functions." + str(call.get("name")) + ":0<|tool_call_argument_begin|>"
                            + json.dumps(call.get("arguments"), ensure_ascii=False) + "<|tool_call_end|><|tool_calls_section_end|>"),
    reasoning_parser="kimi", tool_call_parser="kimi_k2")

LLAMA3 = Family(
    name="llama", bos="<|begin_of_text|>", open=lambda r: f"<|start_header_id|>{'ipython' if r == 'tool' else r}<|end_header_id|>\n\n",
    close="<|eot_id|>", eot="<|eot_id|>", generation_prompt="<|start_header_id|>assistant<|end_header_id|>\n\n",
    tool_call_parser="llama3")

GEMMA = Family(
    name="gemma", bos="<bos>", open=lambda r: f"<start_of_turn>{'model' if r == 'assistant' else 'user'}\n",
    close="<end_of_turn>\n", eot="<end_of_turn>", after_eot="\n", generation_prompt="<start_of_turn>model\n",
    allowed_append_roles=("user", "tool"))

CHATML = Family(
    name="chatml", open=lambda r: f"<|im_start|>{r}\n", close="<|im_end|>\n", eot="<|im_end|>", after_eot="\n",
    generation_prompt="<|im_start|>assistant\n", tool_role="user", wrap_tool=lambda c: f"<tool_response>\n{c}\n</tool_response>")

FAMILIES = {f.name: f for f in (QWEN3, QWEN35, QWEN_NEXT, GLM47, DEEPSEEK, KIMI, LLAMA3, GEMMA, CHATML)}
FAMILIES.update({"default": CHATML, "qwen": QWEN3, "auto": CHATML})


def get_family(name: str) -> Family:
    if name not in FAMILIES:
        raise KeyError(f"unknown chat family {name!r}; known: {sorted(FAMILIES)}")
    return FAMILIES[name]


def guess_family(tokenizer) -> str:
    """Pick a family from the special tokens a tokenizer knows."""
    def has(tok: str) -> bool:
        try:
            v = tokenizer.convert_tokens_to_ids(tok)
        except Exception:
            return False
        return v is not None and v != getattr(tokenizer, "unk_token_id", None) and (not isinstance(v, int) or v >= 0)

    for probe, fam in (("<|im_assistant|>", "kimi"), ("<|observation|>", "glm47"), ("<｜Assistant｜>", "deepseek"),
                       ("<|eot_id|>", "llama"), ("<start_of_turn>", "gemma"), ("<|im_start|>", "qwen3")):
        if has(probe):
            return fam
    return "chatml"


# ---- append-only check ------------------------------------------------------------------------------------------------

def assert_append_only(old: list[dict], new: list[dict], allowed_roles) -> None:
    """`new` must be `old` plus messages of roles that may follow an assistant turn."""
    if len(new) < len(old):
        raise ValueError(f"the new message list is shorter ({len(new)}) than the stored one ({len(old)})")
    for i, (a, b) in enumerate(zip(old, new)):
        if a.get("role") != b.get("role") or _text(a.get("content")) != _text(b.get("content")):
            raise ValueError(f"message {i} differs from the stored conversation: only appending is allowed")
    for m in new[len(old):]:
        if m["role"] not in allowed_roles:
            raise ValueError(f"a {m['role']!r} message cannot be appended (allowed: {sorted(allowed_roles)})")


# ---- comparing a trajectory with a fresh tokenisation (CI check) --------------------------------------------------------

def compare_token_sequences(kept: list[int], fresh: list[int], special_ids: set[int], trailing_ids: set[int] = frozenset()) -> dict:
    """How a token trajectory kept by TITO differs from re-tokenising the rendered conversation.  Differences in ordinary
    text ids are expected (that is why trajectories are kept); a different NUMBER or ORDER of special tokens means the
    format itself went wrong.  Trailing format ids (a final newline) are ignored."""
    def strip(x):
        x = list(x)
        while x and x[-1] in trailing_ids:
            x.pop()
        return x

    a, b = strip(kept), strip(fresh)
    sa, sb = [t for t in a if t in special_ids], [t for t in b if t in special_ids]
    return {"equal": a == b, "special_equal": sa == sb, "special_count_kept": len(sa), "special_count_fresh": len(sb),
            "length_kept": len(a), "length_fresh": len(b),
            "first_diff": next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), None if len(a) == len(b) else min(len(a), len(b)))}
