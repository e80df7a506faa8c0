"""Pipeline parallelism over point-to-point send/recv (NCCL on GPUs, gloo on CPU).

The reference takes Megatron's pipeline schedules (1F1B / interleaved, miles/backends/megatron_utils/model.py:395-411,
507-517) with NCCL p2p between stages; pipeline traffic is one `[tokens, hidden]` activation per micro-batch per
boundary, small next to TP/EP traffic, so it stays on NCCL here as well.  A stage is a `Qwen3Model` built with a
`layer_range` (`models/qwen3.py`): the first stage embeds tokens, the last applies the final norm and head.

Schedules (`--pp-schedule`): `1f1b` (default, `PipeStage.run_1f1b`) is Megatron's non-interleaved order — `pp − rank − 1`
warm-up forwards, then one forward and one backward per step with the two directions exchanged in ONE grouped p2p call,
then the remaining backwards — so a stage keeps at most `pp − rank` micro-batches of activations; `gpipe` runs all
forwards and then all backwards (`recv_forward` / `send_forward` / `backward`), with sends posted asynchronously and
completed before the next send.  With `--virtual-pipeline-model-parallel-size v` every rank owns v model chunks and the
interleaved order runs in `train/step_runner.py` (`InterleavedStepRunner`) over `models/qwen3.py` (`VirtualStages`).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class StageIO:
    """What one micro-batch leaves behind after its forward pass on this stage."""

    hidden_in: torch.Tensor | None     # leaf received from the previous stage (None on the first stage)
    hidden_out: torch.Tensor | None    # tensor sent to the next stage (None on the last stage)


class PipeStage:
    def __init__(self, ps, hidden_size: int, dtype, device):
        self.ps, self.hidden, self.dtype, self.device = ps, hidden_size, dtype, device
        self.prev = ps.pp_ranks[ps.pp_rank - 1] if ps.pp_rank > 0 else None
        self.next = ps.pp_ranks[ps.pp_rank + 1] if ps.pp_rank < ps.pp_size - 1 else None
        self._pending: list = []

    @property
    def is_first(self) -> bool:
        return self.prev is None

    @property
    def is_last(self) -> bool:
        return self.next is None

    def _rows(self, num_tokens: int) -> int:
        """Rows of a boundary activation on this rank: the token axis is sharded under sequence parallelism."""
        ps = self.ps
        return num_tokens // ps.tp_size if (ps.tp_size > 1 and ps.sequence_parallel) else num_tokens

    def _flush(self):
        for w in self._pending:
            w.wait()
        self._pending.clear()

    # ---- forward direction -----------------------------------------------------------------------
    def recv_forward(self, num_tokens: int, requires_grad: bool = True) -> torch.Tensor | None:
        if self.is_first:
            return None
        buf = torch.empty(self._rows(num_tokens), self.hidden, dtype=self.dtype, device=self.device)
        dist.recv(buf, src=self.prev)
        return buf.requires_grad_(requires_grad)

    def send_forward(self, hidden: torch.Tensor):
        if self.is_last:
            return
        self._flush()
        self._pending.append(dist.isend(hidden.detach().contiguous(), dst=self.next))

    # ---- backward direction ------------------------------------------------------------------------
    def backward(self, io: StageIO, loss: torch.Tensor | None = None):
        """Run this stage's backward for one micro-batch: from `loss` on the last stage, else from the gradient
        received from the next stage; then pass the input gradient upstream."""
        if self.is_last:
            assert loss is not None
            loss.backward()
        else:
            g = torch.empty_like(io.hidden_out)
            dist.recv(g, src=self.next)
            io.hidden_out.backward(g)
        if not self.is_first:
            self._flush()
            grad = io.hidden_in.grad if io.hidden_in.grad is not None else torch.zeros_like(io.hidden_in)
            self._pending.append(dist.isend(grad.contiguous(), dst=self.prev))

    def finish(self):
        self._flush()

    # ---- one-forward-one-backward schedule ---------------------------------------------------------
    def _exchange(self, send: tuple | None, recv: tuple | None):
        """One grouped p2p call: (tensor, peer) to send and (buffer, peer) to receive.  Grouping the two directions is
        what keeps neighbouring stages from waiting on each other's sends (NCCL matches the whole group at once)."""
        ops = []
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send[0], send[1]))
        if recv is not None:
            ops.append(dist.P2POp(dist.irecv, recv[0], recv[1]))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def run_1f1b(self, n_micro: int, num_tokens_of, forward_step):
        """Megatron's non-interleaved 1F1B order: `pp − rank − 1` warm-up forwards, then one forward and one backward per
        step, then the remaining backwards — at most `pp − rank` micro-batches of activations are alive on a stage.
        forward_step(i, hidden_in) → (hidden_out, loss): hidden_out is None on the last stage, loss None elsewhere."""
        self._flush()
        warm = min(self.ps.pp_size - self.ps.pp_rank - 1, n_micro)
        rem = n_micro - warm
        alive: list[tuple] = []

        def buf(i):
            return torch.empty(self._rows(num_tokens_of(i)), self.hidden, dtype=self.dtype, device=self.device)

        def backward(entry, g):
            hidden_in, hidden_out, loss = entry
            if self.is_last:
                loss.backward()
            else:
                hidden_out.backward(g)
            if self.is_first:
                return None
            return (hidden_in.grad if hidden_in.grad is not None else torch.zeros_like(hidden_in)).contiguous()

        grad_on = torch.is_grad_enabled()
        x = None
        for i in range(warm):
            if not self.is_first:
                x = buf(i)
                self._exchange(None, (x, self.prev))
                x.requires_grad_(grad_on)
            out, loss = forward_step(i, x)
            self._exchange((out.detach().contiguous(), self.next), None)
            alive.append((x, out, loss))
        if rem > 0 and not self.is_first:
            x = buf(warm)
            self._exchange(None, (x, self.prev))
            x.requires_grad_(grad_on)
        for i in range(rem):
            out, loss = forward_step(warm + i, x)
            alive.append((x, out, loss))
            g = None
            if not self.is_last:
                g = torch.empty_like(alive[0][1])            # the gradient coming back belongs to the oldest micro-batch alive
                self._exchange((out.detach().contiguous(), self.next), (g, self.next))
            gin = backward(alive.pop(0), g)
            nxt = None
            if i + 1 < rem and not self.is_first:
                nxt = buf(warm + i + 1)
            if not self.is_first:
                self._exchange((gin, self.prev), (nxt, self.prev) if nxt is not None else None)
                if nxt is not None:
                    nxt.requires_grad_(grad_on)
            x = nxt
        for _ in range(warm):
            entry = alive.pop(0)
            g = torch.empty_like(entry[1])
            self._exchange(None, (g, self.next))
            gin = backward(entry, g)
            if not self.is_first:
                self._exchange((gin, self.prev), None)


def broadcast_from_last_stage(t: torch.Tensor, ps) -> torch.Tensor:
    """Metrics and per-token results exist on the last stage only; share them with the other stages of the pipeline."""
    if ps.pp_size == 1:
        return t
    dist.broadcast(t, src=ps.pp_ranks[-1], group=ps.pp_group)
    return t
