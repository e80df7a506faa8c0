"""Fully asynchronous rollout: a persistent producer keeps the engines busy across trainer steps and weight updates.

Behaviour of the reference's fully-async mode (miles/rollout/fully_async_rollout.py, fully_async_data_buffer.py:77-347,
submission_scheduler.py:16-71): generation never drains; finished prompt groups wait in a buffer; the trainer takes
`rollout_batch_size` groups per step; a group whose oldest tokens were sampled more than `--max-weight-staleness`
versions ago is dropped (or regenerated, `--staleness-policy retry`).  Weight updates pause the engine between two
decode steps, so one trajectory may span several weight versions — its `weight_versions` spans record which.

    --rollout-function-path miles_b200.rollout.fully_async.FullyAsyncRolloutFn

The producer runs its own event loop in a thread; the trainer thread blocks in `__call__` only while the buffer is
short of fresh groups.
"""
from __future__ import annotations

import asyncio
import threading
import time
from collections import deque

from ..types import Sample, Status
from ..utils.misc import load_function
from .inference_rollout import (InferenceRolloutFn, RolloutFnEvalInput, RolloutFnTrainOutput, _State,
                                generate_and_rm_group)


def group_oldest_version(group: list[Sample]) -> int | None:
    vs = [s.oldest_weight_version for s in group if s.oldest_weight_version is not None]
    return min(vs) if vs else None


class StalenessBuffer:
    """Thread-safe FIFO of finished groups with staleness accounting."""

    def __init__(self, max_staleness: int | None, policy: str = "drop"):
        assert policy in ("drop", "retry", "keep")
        self.max_staleness, self.policy = max_staleness, policy
        self.q: deque[list[Sample]] = deque()
        self.cv = threading.Condition()
        self.stats = {"put": 0, "taken": 0, "dropped_stale": 0, "retried": 0}
        self.retry: deque[list[Sample]] = deque()

    def __len__(self):
        with self.cv:
            return len(self.q)

    def put(self, group: list[Sample]):
        with self.cv:
            self.q.append(group)
            self.stats["put"] += 1
            self.cv.notify_all()

    def _fresh(self, group, current_version: int) -> bool:
        if self.max_staleness is None or self.policy == "keep":
            return True
        v = group_oldest_version(group)
        return v is None or current_version - v <= self.max_staleness

    def _evict_stale(self, current_version: int):
        kept = deque()
        for g in self.q:
            if self._fresh(g, current_version):
                kept.append(g)
            else:
                self.stats["dropped_stale"] += 1
                if self.policy == "retry":
                    self.retry.append(g)
                    self.stats["retried"] += 1
        self.q = kept

    def take(self, n: int, current_version: int, timeout: float | None = None, alive=lambda: True) -> list[list[Sample]]:
        """Block until n fresh groups are available (stale ones are evicted while waiting)."""
        deadline = None if timeout is None else time.time() + timeout
        with self.cv:
            while True:
                self._evict_stale(current_version)
                if len(self.q) >= n:
                    out = [self.q.popleft() for _ in range(n)]
                    self.stats["taken"] += n
                    return out
                if not alive():
                    raise RuntimeError("fully-async producer stopped before the buffer filled")
                wait = 0.5 if deadline is None else min(0.5, deadline - time.time())
                if wait <= 0:
                    raise TimeoutError(f"buffer holds {len(self.q)} of {n} fresh groups")
                self.cv.wait(wait)

    def pop_retries(self) -> list[list[Sample]]:
        with self.cv:
            out = list(self.retry)
            self.retry.clear()
            return out


class SubmissionScheduler:
    """How many prompt groups may be in flight: enough to refill the buffer to `target_buffered` plus one batch,
    never more than `max_inflight` (back-pressure keeps staleness bounded when the trainer is the slow side)."""

    def __init__(self, batch: int, max_inflight: int, target_buffered: int):
        self.batch, self.max_inflight, self.target_buffered = batch, max_inflight, target_buffered

    def allowance(self, inflight: int, buffered: int) -> int:
        want = self.target_buffered + self.batch - buffered - inflight
        return max(0, min(want, self.max_inflight - inflight))


class FullyAsyncRolloutFn:
    def __init__(self, args, data_source, client, eval_sources=None):
        self.args, self.data_source, self.client = args, data_source, client
        self.inner = InferenceRolloutFn(args, data_source, client, eval_sources)
        self.buffer = StalenessBuffer(getattr(args, "max_weight_staleness", None), getattr(args, "staleness_policy", "drop"))
        batch = args.rollout_batch_size
        inflight = getattr(args, "over_sampling_batch_size", None) or batch
        self.scheduler = SubmissionScheduler(batch, max(inflight, batch), getattr(args, "fully_async_buffer_groups", None) or batch)
        self.weight_version = 0
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self._error: BaseException | None = None
        f = getattr(args, "dynamic_sampling_filter_path", None)
        self.dynamic_filter = load_function(f) if f else None
        self.dropped_filter = 0

    # ---- producer ----------------------------------------------------------------------------------
    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="fully-async-rollout", daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=30)
            self._thread = None

    def alive(self) -> bool:
        return self._thread is not None and self._thread.is_alive() and self._error is None

    def _run(self):
        try:
            asyncio.run(self._producer())
        except BaseException as e:  # surfaces in the trainer thread on its next take()
            self._error = e

    async def _producer(self):
        args = self.args
        state = _State()
        sp = self.inner.sampling_params()
        pending: set[asyncio.Task] = set()
        await self.client.begin()
        try:
            while not self._stop.is_set():
                allow = self.scheduler.allowance(len(pending), len(self.buffer))
                groups = self.buffer.pop_retries()[:allow]
                for g in groups:                     # regenerate stale groups from their prompts
                    for s in g:
                        _reset_sample(s)
                if allow - len(groups) > 0:
                    groups += self.data_source.get_samples(allow - len(groups))
                for g in groups:
                    pending.add(asyncio.ensure_future(generate_and_rm_group(args, g, sp, self.client, state)))
                if not pending:
                    await asyncio.sleep(0.005)
                    continue
                finished, pending = await asyncio.wait(pending, timeout=0.05, return_when=asyncio.FIRST_COMPLETED)
                for t in finished:
                    group = t.result()
                    if any(s.status == Status.ABORTED for s in group):
                        continue
                    if self.dynamic_filter is not None and not self.dynamic_filter(args, group):
                        self.dropped_filter += 1
                        continue
                    self.buffer.put(group)
        finally:
            state.aborted = True
            if pending:
                await self.client.abort_all()
                await asyncio.gather(*pending, return_exceptions=True)
            await self.client.finish()

    # ---- trainer side ------------------------------------------------------------------------------
    def set_weight_version(self, v: int):
        self.weight_version = int(v)

    def __call__(self, inp):
        if isinstance(inp, RolloutFnEvalInput):
            raise NotImplementedError("evaluate through --eval-function-path with a drained engine")
        self.start()
        if self._error is not None:
            raise RuntimeError("fully-async producer failed") from self._error
        t0 = time.time()
        groups = self.buffer.take(self.args.rollout_batch_size, self.weight_version,
                                  timeout=getattr(self.args, "fully_async_take_timeout", None), alive=self.alive)
        if self._error is not None:
            raise RuntimeError("fully-async producer failed") from self._error
        stale = [self.weight_version - v for v in (group_oldest_version(g) for g in groups) if v is not None]
        n_tok = sum(s.response_length for g in groups for s in g)
        dt = time.time() - t0
        metrics = {"rollout/staleness/mean": sum(stale) / len(stale) if stale else 0.0,
                   "rollout/staleness/max": float(max(stale)) if stale else 0.0,
                   "rollout/dropped_stale": float(self.buffer.stats["dropped_stale"]),
                   "rollout/dynamic_filter_dropped": float(self.dropped_filter),
                   "rollout/buffered_groups": float(len(self.buffer)),
                   "perf/rollout_wait_time": dt, "perf/rollout_tokens_per_sec": n_tok / max(dt, 1e-9)}
        return RolloutFnTrainOutput(groups, metrics)


def _reset_sample(s: Sample):
    """Back to the bare prompt (retry policy)."""
    p = s.prompt_length
    s.tokens = list(s.tokens[:p])
    s.response, s.response_length, s.loss_mask, s.rollout_log_probs = "", 0, None, None
    s.rollout_routed_experts, s.weight_versions, s.reward, s.status = None, [], None, Status.PENDING
