"""Token-in-token-out chat tokenisation: extend a token trajectory by new messages without re-tokenising what exists.

Why: an agent framework speaks a chat API (lists of text messages).  If every turn re-renders and re-tokenises the
whole conversation, the ids of earlier *model-generated* text can change (BPE merges differ across boundaries, special
tokens typed as text, trailing whitespace), and the trainer would then score tokens the engine never sampled.  The
reference solves this with an incremental, per-model-family tokenizer (miles/utils/chat_template_utils/
tito_tokenizer.py:99-1247); the contract kept here:

* ids already in the trajectory are never touched;
* a new non-assistant message contributes exactly the ids of `render(prefix + message) − render(prefix)` (text suffix
  of the chat template), tokenised on its own;
* an assistant turn contributes the engine's ids verbatim, followed by the template's end-of-turn ids if the engine
  stopped before emitting them.

Families differ in their templates; the generic path asks the HF tokenizer's own `apply_chat_template`, and a built-in
ChatML renderer (Qwen family) covers tokenizers without a template.
"""
from __future__ import annotations

from typing import Any


def chatml_render(messages: list[dict], add_generation_prompt: bool = False, tools: list | None = None) -> str:
    out = []
    for m in messages:
        role, content = m["role"], m.get("content") or ""
        if role == "tool":
            out.append(f"<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n")
        else:
            out.append(f"<|im_start|>{role}\n{content}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
    return "".join(out)


class TitoTokenizer:
    def __init__(self, tokenizer, family: str = "auto", end_of_turn: str | None = None):
        self.tok = tokenizer
        self.family = family
        has_template = getattr(tokenizer, "chat_template", None) is not None
        self.use_builtin = family in ("chatml", "qwen") or (family == "auto" and not has_template)
        self.end_of_turn = end_of_turn if end_of_turn is not None else "<|im_end|>\n"

    # ---- rendering / encoding ---------------------------------------------------------------------
    def render(self, messages: list[dict], add_generation_prompt: bool = False, tools: list | None = None) -> str:
        if self.use_builtin:
            return chatml_render(messages, add_generation_prompt, tools)
        return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt, tools=tools)

    def encode(self, text: str) -> list[int]:
        out = self.tok(text, add_special_tokens=False)
        return list(out["input_ids"] if isinstance(out, dict) or hasattr(out, "keys") else out)

    # ---- incremental steps --------------------------------------------------------------------------
    def start(self, messages: list[dict], tools: list | None = None) -> list[int]:
        """Ids of a fresh conversation up to and including the assistant generation prompt."""
        return self.encode(self.render(messages, add_generation_prompt=True, tools=tools))

    def extend(self, prev_messages: list[dict], new_messages: list[dict], tools: list | None = None) -> list[int]:
        """Ids to append after an assistant turn for `new_messages` (tool results, user turns) plus the next
        generation prompt.  Only the text suffix is tokenised."""
        before = self.render(prev_messages, add_generation_prompt=False, tools=tools)
        after = self.render(prev_messages + new_messages, add_generation_prompt=True, tools=tools)
        assert after.startswith(before), "chat template is not prefix-stable; use a family-specific renderer"
        return self.encode(after[len(before):])

    def close_assistant_turn(self, generated_ids: list[int]) -> list[int]:
        """Template ids that must follow the model's own ids to end its turn (empty when the model emitted them)."""
        eot = self.encode(self.end_of_turn)
        if not eot:
            return []
        first = eot[0]                               # e.g. <|im_end|>; the rest is template whitespace
        if generated_ids and generated_ids[-1] == first:
            return eot[1:]
        if len(generated_ids) >= len(eot) and generated_ids[-len(eot):] == eot:
            return []
        return eot

    def decode(self, ids: list[int]) -> str:
        return self.tok.decode(ids)


class ByteChatTokenizer:
    """Self-contained tokenizer for tests and smoke runs: UTF-8 bytes (ids 0–255) plus ChatML specials."""

    SPECIALS = {"<|im_start|>": 256, "<|im_end|>": 257, "<|endoftext|>": 258}
    chat_template = None
    eos_token_id = 257
    vocab_size = 259

    def __call__(self, text: str, add_special_tokens: bool = False) -> dict[str, Any]:
        ids, i = [], 0
        while i < len(text):
            for s, t in self.SPECIALS.items():
                if text.startswith(s, i):
                    ids.append(t)
                    i += len(s)
                    break
            else:
                ids.extend(text[i].encode("utf-8"))
                i += 1
        return {"input_ids": ids}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        inv = {v: k for k, v in self.SPECIALS.items()}
        out, buf = [], bytearray()
        for t in ids:
            if t in inv:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
                if not skip_special_tokens:
                    out.append(inv[t])
            else:
                buf.append(int(t) % 256)
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)
