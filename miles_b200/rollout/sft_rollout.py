"""Supervised fine-tuning through the rollout interface: nothing is generated, the "rollout" tokenises conversations and
marks which tokens are trained on.

Reference: miles/rollout/sft_rollout.py:16-68 (reads a batch from the data buffer, `MultiTurnLossMaskGenerator` builds
token ids and the loss mask, reward 0) and miles/utils/mask_utils.py (per-family mask generators).  A sample's `prompt` is
either a message list (`[{"role": …, "content": …}, …]`, any number of turns, optional `tools` in the metadata) or a
plain string with the answer in `label`.  The loss mask is 1 on the tokens of every ASSISTANT turn — its content and the
end-of-turn token the model must learn to emit — and 0 on system / user / tool text and on the format text that opens a
turn.  Turns are rendered one by one with the chat family's fixed renderer (`session/tito_families.py`), so the mask is
exact by construction instead of being recovered by searching the rendered text.

Use with `--loss-type sft_loss --rollout-function-path miles_b200.rollout.sft_rollout.SftRolloutFn`.
"""
from __future__ import annotations

from ..session.tito import TitoTokenizer
from ..types import Sample, Status
from .inference_rollout import RolloutFnTrainInput, RolloutFnTrainOutput


def conversation_tokens_and_mask(tito: TitoTokenizer, messages: list[dict], tools: list | None = None) -> tuple[list[int], list[int]]:
    """(token ids, loss mask) of a whole conversation; mask 1 = assistant-produced tokens including the turn's closing token."""
    spec = tito.spec
    ids: list[int] = []
    mask: list[int] = []

    def add(text: str, m: int):
        if text:
            t = tito.encode(text)
            ids.extend(t)
            mask.extend([m] * len(t))

    # the head (bos, system prompt with tool schemas) comes from the renderer itself
    head_msgs = [messages[0]] if messages and messages[0]["role"] == "system" else []
    add(spec.render(head_msgs, False, tools), 0)
    rest = messages[len(head_msgs):]
    i = 0
    while i < len(rest):
        m = rest[i]
        if m["role"] == "assistant":
            whole = spec.message(m)
            opener = spec.open("assistant")
            body = whole[len(opener):]
            # the closing token belongs to the model; format text after it (Qwen's newline) does not
            tail = spec.after_eot if spec.after_eot and body.endswith(spec.after_eot) else ""
            add(opener, 0)
            add(body[: len(body) - len(tail)] if tail else body, 1)
            add(tail, 0)
            i += 1
        elif m["role"] == "tool" and spec.extra.get("group_tool_results"):
            j = i
            while j < len(rest) and rest[j]["role"] == "tool":
                j += 1
            add(spec.render(rest[i:j]), 0) if not spec.bos else add(spec.render(rest[i:j])[len(spec.bos):], 0)
            i = j
        else:
            add(spec.message(m), 0)
            i += 1
    if spec.stop_role_tags and messages and messages[-1]["role"] == "assistant":
        # families that end a turn with the next role tag: the model must emit it, so it is appended and trained on
        add(spec.stop_role_tags[0], 1)
    return ids, mask


class SftRolloutFn:
    def __init__(self, args, data_source, client=None, eval_sources=None):
        self.args, self.data_source = args, data_source
        tok = getattr(data_source, "tokenizer", None)
        if tok is None:
            from ..orchestration.wiring import load_tokenizer

            tok = load_tokenizer(args)
        assert tok is not None, "SFT needs a tokenizer (--hf-checkpoint or --tokenizer-path)"
        family = getattr(args, "tito_model", None) or "default"
        if family == "default":                          # --loss-mask-type names the family in the reference's vocabulary
            family = {"qwen": "chatml", "qwen3": "qwen3", "distill_qwen": "qwen3"}.get(getattr(args, "loss_mask_type", None) or "", "auto")
        self.tito = TitoTokenizer(tok, family)
        self.tito.use_template = False                       # masks need the per-turn renderer
        self.max_len = getattr(args, "rollout_max_context_len", None)

    def __call__(self, inp):
        assert isinstance(inp, RolloutFnTrainInput), "the SFT rollout has no evaluation mode"
        groups = self.data_source.get_samples(self.args.rollout_batch_size)
        dropped = 0
        out = []
        for group in groups:
            kept = []
            for s in group:
                messages = s.prompt if isinstance(s.prompt, list) else \
                    [{"role": "user", "content": s.prompt}, {"role": "assistant", "content": s.label or ""}]
                ids, mask = conversation_tokens_and_mask(self.tito, messages, (s.metadata or {}).get("tools"))
                if self.max_len and len(ids) > self.max_len:
                    ids, mask = ids[: self.max_len], mask[: self.max_len]
                if 1 not in mask:
                    dropped += 1
                    continue
                first = mask.index(1)
                s.tokens, s.response_length = ids, len(ids) - first
                s.loss_mask = mask[first:]
                s.reward, s.status = 0.0, Status.COMPLETED
                s.rollout_log_probs = None
                kept.append(s)
            if kept:
                out.append(kept)
        return RolloutFnTrainOutput(out, {"rollout/sft_dropped": float(dropped)})
