"""Training-side profiling: torch-profiler windows over whole rollouts or over the inner loops, allocator history dumps,
and NVTX ranges around the trainer's phases.

Same switches as the reference's `TrainProfiler` (miles/utils/profile_utils.py:13-147): `--use-pytorch-profiler` with
`--profile-target {train_overall, train_actor, train_log_probs}` and the step window `--profile-step-start/-end` (traces go
to `--tensorboard-dir`, one worker name per target and rank); `--record-memory-history` with `--memory-snapshot-dir`,
`--memory-snapshot-path`, `--memory-snapshot-num-steps` (a snapshot is also dumped when an allocation fails).  NVTX ranges
(`--nvtx`) are cheap markers that `ncu` / CUPTI tools show on the timeline; they are no-ops without CUDA.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Iterable, Iterator

import torch


def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _make_profiler(args, name: str):
    start, end = int(getattr(args, "profile_step_start", 0) or 0), int(getattr(args, "profile_step_end", 1) or 1)
    out_dir = getattr(args, "tensorboard_dir", None) or "profiler_traces"
    os.makedirs(out_dir, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    return torch.profiler.profile(
        activities=acts,
        schedule=torch.profiler.schedule(wait=max(start - 1, 0), warmup=1 if start > 0 else 0, active=max(end - start, 1), repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(out_dir, worker_name=f"{name}_rank_{_rank()}", use_gzip=True),
        record_shapes=True, with_stack=bool(getattr(args, "profile_with_stack", True)), profile_memory=True, with_flops=True)


class _MemoryHistory:
    """Allocator event history (`torch.cuda.memory._record_memory_history`) dumped after N rollouts and on allocation failure."""

    def __init__(self, args):
        d = getattr(args, "memory_snapshot_dir", None) or "."
        os.makedirs(d, exist_ok=True)
        self.path = os.path.join(d, f"memory_snapshot_time{time.time():.0f}_rank{_rank()}_{getattr(args, 'memory_snapshot_path', 'snapshot.pickle')}")
        self.active = False

    def start(self):
        if not torch.cuda.is_available():
            return
        torch.cuda.memory._record_memory_history(max_entries=1_000_000, stacks="all")
        self.active = True

        def on_oom(device, alloc, device_alloc, device_free):
            torch.cuda.memory._dump_snapshot(self.path)

        try:
            torch._C._cuda_attach_out_of_memory_observer(on_oom)
        except Exception:
            pass

    def stop(self):
        if not self.active:
            return
        torch.cuda.memory._dump_snapshot(self.path)
        torch.cuda.memory._record_memory_history(enabled=None)
        self.active = False


class TrainProfiler:
    def __init__(self, args):
        self.args = args
        targets = set(getattr(args, "profile_target", None) or ["train_overall"])
        self.targets = targets
        self.overall = _make_profiler(args, "train_overall") if getattr(args, "use_pytorch_profiler", False) and "train_overall" in targets else None
        self.memory = None
        if getattr(args, "record_memory_history", False) and "train_overall" in targets:
            self.memory = _MemoryHistory(args)
            self.memory.start()
        self.nvtx = bool(getattr(args, "nvtx", False)) and torch.cuda.is_available()

    def on_init_end(self):
        if self.overall is not None:
            self.overall.start()

    def step(self, rollout_id: int):
        if self.overall is not None:
            with contextlib.suppress(RuntimeError):       # the scheduled window is over and the profiler stopped itself
                self.overall.step()
        n = getattr(self.args, "memory_snapshot_num_steps", None)
        if self.memory is not None and n is not None and rollout_id == n - 1:
            self.memory.stop()

    def finish(self):
        if self.overall is not None:
            with contextlib.suppress(Exception):
                self.overall.stop()
        if self.memory is not None:
            self.memory.stop()

    def iterate(self, name: str, iterator: Iterable) -> Iterator:
        """Wrap an inner loop (`train_actor`: optimizer steps, `train_log_probs`: forward-only micro-batches) in its own
        profiler window when that target is selected."""
        # one Kineto session at a time: with `train_overall` selected the inner loops are already inside its window
        if not (getattr(self.args, "use_pytorch_profiler", False) and name in self.targets) or self.overall is not None:
            yield from iterator
            return
        prof = _make_profiler(self.args, name)
        prof.start()
        try:
            for item in iterator:
                yield item
                with contextlib.suppress(RuntimeError):
                    prof.step()
        finally:
            with contextlib.suppress(Exception):
                prof.stop()

    @contextlib.contextmanager
    def range(self, name: str):
        """NVTX range around a phase (no-op unless `--nvtx` and CUDA)."""
        if not self.nvtx:
            yield
            return
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
