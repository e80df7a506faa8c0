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


class InterleavedStepRunner(_Base):
    """Virtual pipeline (`--virtual-pipeline-model-parallel-size v`): every rank owns v model chunks (`models.qwen3.VirtualStages`)
    and runs Megatron's interleaved one-forward-one-backward order (reference: the interleaved schedule the trainer takes from
    Megatron, miles/backends/megatron_utils/model.py:395-411).  Unit k of a direction is the same (micro-batch, chunk) on
    every rank — chunk (k // pp) % v, micro-batch (k // (pp·v))·pp + k % pp, chunks reversed for backward — so on each
    communicator every ordered pair of ranks carries one stream in one order and a blocking receive before a unit plus an
    asynchronous send after it cannot deadlock.  Warm-up is (pp − rank − 1)·2 + (v − 1)·pp forward units, then one forward
    and one backward per step, then the remaining backwards."""

    def _geometry(self, n_micro: int):
        ps = self.actor.ps
        pp, v = ps.pp_size, ps.vpp_size
        assert n_micro % pp == 0, f"the interleaved schedule needs a multiple of {pp} micro-batches per step, got {n_micro}"
        return pp, v, n_micro * v

    @staticmethod
    def _unit(k: int, pp: int, v: int, forward: bool):
        c = (k // pp) % v
        return (k // (pp * v)) * pp + k % pp, (c if forward else v - 1 - c)

    def _rows(self, n_tokens: int) -> int:
        ps = self.actor.ps
        return n_tokens // ps.tp_size if (ps.tp_size > 1 and ps.sequence_parallel) else n_tokens

    def _run(self, micro_batches, pack, on_last, *, replay: bool, backward: bool):
        import torch
        import torch.distributed as dist

        a = self.actor
        ps = a.ps
        pp, v, total = self._geometry(len(micro_batches))
        r = ps.pp_rank
        nxt, prv = ps.pp_ranks[(r + 1) % pp], ps.pp_ranks[(r - 1) % pp]
        fwd_g, bwd_g = ps.pp_fwd_group, ps.pp_bwd_group
        hidden, dtype, dev = a.cfg.hidden_size, next(a.model.parameters()).dtype, a.device
        packed: dict[int, Any] = {}
        alive: dict[tuple, tuple] = {}
        sends: list = []
        grad_on = torch.is_grad_enabled() and backward

        def get(i):
            if i not in packed:
                packed[i] = pack(micro_batches[i])
            return packed[i]

        def first_virtual(c):
            return r == 0 and c == 0

        def last_virtual(c):
            return r == pp - 1 and c == v - 1

        def fwd(k):
            i, c = self._unit(k, pp, v, True)
            pb = get(i)
            x = None
            if not first_virtual(c):
                x = torch.empty(self._rows(pb.tokens.numel()), hidden, dtype=dtype, device=dev)
                dist.recv(x, src=prv, group=fwd_g)
                x.requires_grad_(grad_on)
            out = a.model(pb.tokens, a._meta(pb, replay), hidden_in=x, chunk=c)
            if last_virtual(c):
                res = on_last(pb, micro_batches[i], out)
                alive[(i, c)] = (x, None, res)
            else:
                t = out.detach().contiguous()
                sends.append((dist.isend(t, dst=nxt, group=fwd_g), t))
                alive[(i, c)] = (x, out if grad_on else None, None)

        def bwd(k):
            i, c = self._unit(k, pp, v, False)
            x, out, loss = alive.pop((i, c))
            if last_virtual(c):
                loss.backward()
            else:
                g = torch.empty_like(out)
                dist.recv(g, src=nxt, group=bwd_g)
                out.backward(g)
            if not first_virtual(c):
                gin = (x.grad if x.grad is not None else torch.zeros_like(x)).contiguous()
                sends.append((dist.isend(gin, dst=prv, group=bwd_g), gin))
            if all(key[0] != i for key in alive):
                packed.pop(i, None)

        if not backward:
            for k in range(total):
                fwd(k)
                i, c = self._unit(k, pp, v, True)
                alive.pop((i, c), None)
        else:
            warm = min(total, (pp - r - 1) * 2 + (v - 1) * pp)
            for k in range(warm):
                fwd(k)
            for k in range(total - warm):
                fwd(warm + k)
                bwd(k)
            for k in range(total - warm, total):
                bwd(k)
        for w, _ in sends:
            w.wait()

    def forward_only_step(self, micro_batches, pack, compute, *, replay=False):
        import torch

        from ..parallel.pp import broadcast_from_last_stage

        a = self.actor
        ps = a.ps
        results: dict[int, Any] = {}
        micro_batches = list(micro_batches)
        pad = (-len(micro_batches)) % ps.pp_size                 # empty micro-batches keep the unit order regular
        padded = micro_batches + [[] for _ in range(pad)]
        packs: dict[int, Any] = {}

        def pack_keep(idx):
            pb = pack(idx)
            packs[id(idx)] = pb
            return pb

        def on_last(pb, idx, hidden_out):
            lp, _ = a._score_hidden(pb, hidden_out, False)
            results[id(idx)] = lp
            return None

        self._run(padded, pack_keep, on_last, replay=replay, backward=False)
        out = []
        for idx in micro_batches:                                # every stage keeps the same record
            pb = packs.get(id(idx)) or pack(idx)
            lp = results.get(id(idx))
            if lp is None:
                lp = torch.zeros(pb.gather_index.numel(), device=a.device)
            lp = broadcast_from_last_stage(lp.float().contiguous(), ps)
            out.append(compute(pb, idx, lp))
        return out

    def forward_backward_step(self, micro_batches, pack, score, *, want_ent, replay):
        a = self.actor
        micro_batches = list(micro_batches)
        pad = (-len(micro_batches)) % a.ps.pp_size
        padded = micro_batches + [[] for _ in range(pad)]

        def on_last(pb, idx, hidden_out):
            out, ent = a._score_hidden(pb, hidden_out, want_ent)
            return score(pb, idx, out, ent)

        self._run(padded, pack, on_last, replay=replay, backward=True)


def build_step_runner(actor) -> StepRunner:
    custom = getattr(actor.args, "custom_step_runner_path", None)
    if custom:
        from ..utils.misc import load_function

        return load_function(custom)(actor)
    if actor.ps.pp_size > 1 and getattr(actor.ps, "vpp_size", 1) > 1:
        return InterleavedStepRunner(actor)
    if actor.ps.pp_size > 1:
        return OneFOneBStepRunner(actor) if getattr(actor.args, "pp_schedule", "1f1b") == "1f1b" else GPipeStepRunner(actor)
    return LinearStepRunner(actor)
