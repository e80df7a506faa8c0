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

Families differ in their formats and in how a turn ends: `tito_families.py` holds a fixed, prefix-stable renderer and the
boundary rule for each (Qwen3 / 3.5 / Next, GLM-4.7, DeepSeek, Kimi, Llama-3, Gemma, plain ChatML); the generic path asks
the HF tokenizer's own `apply_chat_template`.
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


_DUMMY_PREFIX = [{"role": "system", "content": "s"}, {"role": "user", "content": "u"}, {"role": "assistant", "content": "a"}]


class TitoTokenizer:
    """`family`: a name from `tito_families.FAMILIES` (fixed renderer + boundary rule of that model family), `auto` (the
    tokenizer's own chat template when it has one, else a family guessed from its special tokens), or `template` (always
    the tokenizer's template)."""

    def __init__(self, tokenizer, family: str = "auto", end_of_turn: str | None = None, enable_thinking: bool | None = None):
        from .tito_families import get_family, guess_family

        self.tok = tokenizer
        has_template = getattr(tokenizer, "chat_template", None) is not None
        if family in ("chatml", "qwen"):
            family = {"chatml": "chatml", "qwen": "qwen3"}[family]
        self.use_template = family == "template" or (family == "auto" and has_template)
        if family in ("auto", "template"):
            family = guess_family(tokenizer)
        self.family = family
        self.spec = get_family(family)
        self.enable_thinking = enable_thinking
        self.end_of_turn = end_of_turn if end_of_turn is not None else (self.spec.eot + self.spec.after_eot)
        self.allowed_append_roles = set(self.spec.allowed_append_roles)
        self.reasoning_parser, self.tool_call_parser = self.spec.reasoning_parser, self.spec.tool_call_parser
        self._stop_tag_ids = {}
        for tag in self.spec.stop_role_tags:
            ids = self.encode(tag)
            if len(ids) == 1:
                self._stop_tag_ids[ids[0]] = tag

    # ---- rendering / encoding ---------------------------------------------------------------------
    @property
    def use_builtin(self) -> bool:
        return not self.use_template

    def render(self, messages: list[dict], add_generation_prompt: bool = False, tools: list | None = None) -> str:
        if self.use_template:
            return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt, tools=tools)
        return self.spec.render(messages, add_generation_prompt, tools, self.enable_thinking)

    def encode(self, text: str) -> list[int]:
        out = self.tok(text, add_special_tokens=False)
        return list(out["input_ids"] if isinstance(out, dict) or hasattr(out, "keys") else out)

    # ---- incremental steps --------------------------------------------------------------------------
    def start(self, messages: list[dict], tools: list | None = None) -> list[int]:
        """Ids of a fresh conversation up to and including the assistant generation prompt."""
        return self.encode(self.render(messages, add_generation_prompt=True, tools=tools))

    def extend(self, prev_messages: list[dict], new_messages: list[dict], tools: list | None = None,
               pretokenized: list[int] | None = None) -> list[int]:
        """Ids to append after an assistant turn for `new_messages` (tool results, user turns) plus the next generation
        prompt.  Only the text suffix is tokenised; with a family renderer it is rendered against a short dummy prefix, so
        nothing of the real history is re-rendered.  `pretokenized` (the trajectory so far) lets the boundary rule see how
        the model ended its turn."""
        from .tito_families import assert_append_only

        assert_append_only(prev_messages, prev_messages + list(new_messages), self.allowed_append_roles)
        if self.use_template:
            before = self.render(prev_messages, add_generation_prompt=False, tools=tools)
            after = self.render(prev_messages + new_messages, add_generation_prompt=True, tools=tools)
        else:
            before = self.spec.render(_DUMMY_PREFIX, False, None, self.enable_thinking)
            after = self.spec.render(_DUMMY_PREFIX + list(new_messages), True, None, self.enable_thinking)
        assert after.startswith(before), "chat template is not prefix-stable; use a family renderer (--tito-model)"
        ids = self.encode(after[len(before):])
        if pretokenized and ids and pretokenized[-1] in self._stop_tag_ids and ids[0] == pretokenized[-1]:
            ids = ids[1:]            # the model ended its turn by sampling the next role tag: it is in the trajectory already
        return ids

    def close_assistant_turn(self, generated_ids: list[int]) -> list[int]:
        """Format ids that must follow the model's own ids to end its turn (empty when the model emitted them, or when the
        family ends a turn with the next role tag)."""
        if generated_ids and generated_ids[-1] in self._stop_tag_ids:
            return []
        eot = self.encode(self.end_of_turn)
        if not eot:
            return []
        first = eot[0]                               # e.g. <|im_end|>; the rest is format whitespace
        if generated_ids and generated_ids[-1] == first:
            return eot[1:]
        if len(generated_ids) >= len(eot) and generated_ids[-len(eot):] == eot:
            return []
        return eot

    def strip_turn_end(self, generated_ids: list[int]) -> list[int]:
        """The model's ids without the token that ended its turn (for decoding the message text)."""
        enders = set(self._stop_tag_ids) | set(self.encode(self.spec.eot)[:1] if self.spec.eot else [])
        return generated_ids[:-1] if generated_ids and generated_ids[-1] in enders else list(generated_ids)

    def special_ids(self) -> set[int]:
        ids = set(getattr(self.tok, "all_special_ids", None) or [])
        sp = getattr(self.tok, "SPECIALS", None)
        if sp:
            ids |= set(sp.values())
        return ids

    def check_against_fresh(self, messages: list[dict], kept: list[int], tools: list | None = None) -> dict:
        """Compare a kept trajectory with a fresh tokenisation of the rendered conversation (see
        `tito_families.compare_token_sequences`)."""
        from .tito_families import compare_token_sequences

        fresh = self.encode(self.render(messages, add_generation_prompt=False, tools=tools))
        trailing = set(self.encode(self.spec.after_eot)) if self.spec.after_eot else set()
        return compare_token_sequences(kept, fresh, self.special_ids(), trailing)

    def decode(self, ids: list[int]) -> str:
        return self.tok.decode(ids)


class ByteChatTokenizer:
    """Self-contained tokenizer for tests and smoke runs: UTF-8 bytes (ids 0–255) plus ChatML specials (or any other list
    of special-token strings, numbered from 256)."""

    SPECIALS = {"<|im_start|>": 256, "<|im_end|>": 257, "<|endoftext|>": 258}
    chat_template = None
    eos_token_id = 257
    vocab_size = 259

    def __init__(self, specials: list[str] | None = None):
        if specials is not None:
            self.SPECIALS = {s: 256 + i for i, s in enumerate(specials)}
            self.vocab_size = 256 + len(specials)
            self.eos_token_id = 256 + len(specials) - 1

    def convert_tokens_to_ids(self, token: str):
        return self.SPECIALS.get(token)

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
