"""Step runners: who decides in which order micro-batches go forward and backward.

The RL side of the trainer knows how to pack a micro-batch and how to turn log-probs into a loss; the backend side knows
how to execute forwards and backwards — one after the other, or interleaved across pipeline stages.  The seam between the
two is a small protocol (reference: miles/backends/training_utils/torch_native/step_runner.py:14-56 `StepRunner` /
`LinearStepRunner`, the torch-native base actor that every non-Megatron backend builds on, and the pipeline schedules of
miles/backends/megatron_utils/model.py:330-520):

    forward_only_step(micro_batches, pack, compute, replay=…)  → [compute(packed, indices, log_probs)]
    forward_backward_step(micro_batches, pack, score, …)       gradients accumulate; nothing is returned
    zero_grad() / apply_step(lr) → {"grad_norm": …}

`LinearStepRunner` — one micro-batch at a time; `GPipeStepRunner` — all forwards of the stage, then all backwards;
`OneFOneBStepRunner` — warm-up forwards, then one forward / one backward alternating, activations of at most
`pp_size − stage` micro-batches alive.  `--custom-step-runner-path module:factory` builds another one from the actor
(a different model stack, a zero-bubble schedule, …).
"""
from __future__ import annotations

from typing import Any, Callable, Protocol


class StepRunner(Protocol):
    def forward_only_step(self, micro_batches: list, pack: Callable, compute: Callable, *, replay: bool) -> list: ...

    def forward_backward_step(self, micro_batches: list, pack: Callable, score: Callable, *, want_ent: bool, replay: bool) -> None: ...

    def zero_grad(self) -> None: ...

    def apply_step(self, lr: float) -> dict: ...


class _Base:
    def __init__(self, actor):
        self.actor = actor

    def zero_grad(self) -> None:
        self.actor.optimizer.zero_grad()

    def apply_step(self, lr: float) -> dict:
        return self.actor.optimizer.step(lr)


class LinearStepRunner(_Base):
    def forward_only_step(self, micro_batches, pack, compute, *, replay=False):
        a, out = self.actor, []
        for idx in micro_batches:
            pb = pack(idx)
            if a.dumper is not None:
                with a.dumper.phase("fwd_only"):
                    lp, _ = a._forward_logprobs(pb, False, replay)
                    a.dumper.dump("log_probs", lp)
                    a.dumper.step()
            else:
                lp, _ = a._forward_logprobs(pb, False, replay)
            out.append(compute(pb, idx, lp))
        return out

    def forward_backward_step(self, micro_batches, pack, score, *, want_ent, replay):
        a = self.actor
        for idx in micro_batches:
            pb = pack(idx)
            if a.dumper is not None:
                with a.dumper.phase("fwd_bwd"):
                    out, ent = a._forward_logprobs(pb, want_ent, replay)
                    a.dumper.dump("log_probs", out)
            else:
                out, ent = a._forward_logprobs(pb, want_ent, replay)
            score(pb, idx, out, ent).backward()


class GPipeStepRunner(_Base):
    """Pipeline stages: every forward of the step first (boundary activations are sent downstream as they are made), then
    the backwards in the same micro-batch order on every stage."""

    def forward_only_step(self, micro_batches, pack, compute, *, replay=False):
        import torch

        from ..parallel.pp import broadcast_from_last_stage

        a, out = self.actor, []
        for idx in micro_batches:
            pb = pack(idx)
            lp, _, _io = a._forward_logprobs_pp(pb, False, replay)
            if lp is None:
                lp = torch.zeros(pb.gather_index.numel(), device=a.device)
            lp = broadcast_from_last_stage(lp.float().contiguous(), a.ps)      # every stage keeps the same record
            out.append(compute(pb, idx, lp))
        a._pipe().finish()
        return out

    def forward_backward_step(self, micro_batches, pack, score, *, want_ent, replay):
        a = self.actor
        pipelined: list = []
        for idx in micro_batches:
            pb = pack(idx)
            out, ent, io = a._forward_logprobs_pp(pb, want_ent, replay)
            pipelined.append((score(pb, idx, out, ent) if out is not None else None, io))
        stage = a._pipe()
        for loss, io in pipelined:
            stage.backward(io, loss)
        stage.finish()


class OneFOneBStepRunner(GPipeStepRunner):
    def forward_backward_step(self, micro_batches, pack, score, *, want_ent, replay):
        a = self.actor
        stage = a._pipe()
        packed: dict[int, Any] = {}

        def get(i):
            if i not in packed:
                packed[i] = pack(micro_batches[i])
            return packed[i]

        def forward_step(i, hidden_in):
            pb = get(i)
            hidden = a.model(pb.tokens, a._meta(pb, replay), hidden_in=hidden_in)
            if not stage.is_last:
                packed.pop(i, None)
                return hidden, None
            out, ent = a._score_hidden(pb, hidden, want_ent)
            packed.pop(i, None)
            return None, score(pb, micro_batches[i], out, ent)

        stage.run_1f1b(len(micro_batches), lambda i: get(i).tokens.numel(), forward_step)


def build_step_runner(actor) -> StepRunner:
    custom = getattr(actor.args, "custom_step_runner_path", None)
    if custom:
        from ..utils.misc import load_function

        return load_function(custom)(actor)
    if actor.ps.pp_size > 1:
        return OneFOneBStepRunner(actor) if getattr(actor.args, "pp_schedule", "1f1b") == "1f1b" else GPipeStepRunner(actor)
    return LinearStepRunner(actor)
