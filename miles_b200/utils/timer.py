"""Named wall-clock spans and device-side timing.

`Timer` accumulates named host spans (what the reference's `Timer` singleton does,
miles/utils/timer.py:15-99, feeding `perf/*_time`).  `DeviceTimer` measures with CUDA events on the
launching stream and reduces with MAX over ranks — the number every multi-GPU measurement in this
package reports.
"""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch


class Timer:
    def __init__(self):
        self.totals: dict[str, float] = {}
        self._starts: dict[str, float] = {}
        self.sinks: list = []

    def start(self, name: str):
        assert name not in self._starts, f"timer {name} already running"
        self._starts[name] = time.perf_counter()

    def end(self, name: str) -> float:
        dt = time.perf_counter() - self._starts.pop(name)
        self.totals[name] = self.totals.get(name, 0.0) + dt
        for s in self.sinks:
            s(name, dt)
        return dt

    @contextmanager
    def span(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.end(name)

    @contextmanager
    def inverse(self, name: str):
        """Pause an outer running span while the body runs (e.g. `train_wait`)."""
        running = name in self._starts
        if running:
            self.end(name)
        try:
            yield
        finally:
            if running:
                self.start(name)

    def pop_all(self) -> dict[str, float]:
        out, self.totals = self.totals, {}
        return out


_GLOBAL = Timer()


def global_timer() -> Timer:
    return _GLOBAL


class DeviceTimer:
    """CUDA-event timer: `with t.measure(): ...` then `t.ms(group)` = max over ranks of the total."""

    def __init__(self):
        self.pairs: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []

    @contextmanager
    def measure(self, stream=None):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        try:
            yield
        finally:
            e.record(stream)
            self.pairs.append((s, e))

    def ms(self, group=None, reduce_max: bool = True) -> float:
        torch.cuda.synchronize()
        total = sum(s.elapsed_time(e) for s, e in self.pairs)
        self.pairs = []
        if reduce_max:
            import torch.distributed as dist

            if dist.is_initialized() and dist.get_world_size(group) > 1:
                t = torch.tensor([total], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                total = float(t.item())
        return total
