"""Pipeline parallelism over point-to-point send/recv (NCCL on GPUs, gloo on CPU).

The reference takes Megatron's pipeline schedules (1F1B / interleaved, miles/backends/megatron_utils/model.py:395-411,
507-517) with NCCL p2p between stages; pipeline traffic is one `[tokens, hidden]` activation per micro-batch per
boundary, small next to TP/EP traffic, so it stays on NCCL here as well.  A stage is a `Qwen3Model` built with a
`layer_range` (`models/qwen3.py`): the first stage embeds tokens, the last applies the final norm and head.

Schedule: all-forward-then-all-backward over the micro-batches of an optimizer step (GPipe order).  Activations of
a stage live only at its boundaries plus what autograd keeps; with `--recompute-granularity full` that is one
`[tokens, hidden]` tensor per layer per micro-batch.  Sends are posted asynchronously (`isend`) and completed before
the next use of the buffer, receives block: with every stage walking the micro-batches in the same order the
schedule cannot deadlock.
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


def broadcast_from_last_stage(t: torch.Tensor, ps) -> torch.Tensor:
    """Metrics and per-token results exist on the last stage only; share them with the other stages of the pipeline."""
    if ps.pp_size == 1:
        return t
    dist.broadcast(t, src=ps.pp_ranks[-1], group=ps.pp_group)
    return t
