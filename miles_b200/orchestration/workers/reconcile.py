"""Level-triggered reconciliation.

A SOURCE emits events about objects (a full replacement of the known world first, then upserts and deletes); the loop
keeps them in a store indexed by a parent key (for workers: the cell), and every parent whose objects changed is handed
ONCE to the `reconcile(parent_key)` callback, which re-derives what should be done from the store's current contents —
never from the event itself, so a missed or duplicated event cannot leave the system wrong.  Failed reconciles retry
with exponential back-off; a periodic resync re-queues everything; a source stream that ends or fails is reopened.
A simpler polling variant diffs successive listings.

Reference: miles/utils/workers/reconcile/loop.py:26-139 (store + work queue + retry scheduler + stream driver),
retry_scheduler.py:23-74, work_queue.py:12-35, polling_reconcile_loop.py:14-53.
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass
from typing import Any, AsyncIterator, Awaitable, Callable, Hashable


@dataclass(frozen=True)
class Replace:
    """The whole world as the source sees it now; everything not listed is gone."""

    objects: tuple


@dataclass(frozen=True)
class Upsert:
    obj: Any


@dataclass(frozen=True)
class Delete:
    key: Hashable


class WorkQueue:
    """Keys wait at most once however often they are added; `get` returns None after shutdown."""

    def __init__(self):
        self._order: list = []
        self._pending: set = set()
        self._event = asyncio.Event()
        self._closed = False

    def add(self, key) -> None:
        if self._closed or key in self._pending:
            return
        self._pending.add(key)
        self._order.append(key)
        self._event.set()

    async def get(self):
        while not self._order:
            if self._closed:
                return None
            self._event.clear()
            await self._event.wait()
        key = self._order.pop(0)
        self._pending.discard(key)
        return key

    def shutdown(self) -> None:
        self._closed = True
        self._event.set()

    def __len__(self):
        return len(self._order)


class RetryScheduler:
    """Re-adds a failed key after base · 2^(failures−1) seconds, capped; success forgets the history."""

    def __init__(self, on_retry: Callable[[Any], None], base_delay: float = 1.0, max_delay: float = 60.0, clock=time.monotonic):
        self.on_retry, self.base, self.max, self.clock = on_retry, base_delay, max_delay, clock
        self.failures: dict = {}
        self.due: dict = {}

    def delay_of(self, key) -> float:
        n = self.failures.get(key, 0)
        return 0.0 if n == 0 else min(self.max, self.base * (2 ** (n - 1)))

    def note_failure(self, key) -> float:
        self.failures[key] = self.failures.get(key, 0) + 1
        d = self.delay_of(key)
        self.due[key] = self.clock() + d
        return d

    def note_success(self, key) -> None:
        self.failures.pop(key, None)
        self.due.pop(key, None)

    def release_due(self) -> list:
        now = self.clock()
        ready = [k for k, t in self.due.items() if t <= now]
        for k in ready:
            del self.due[k]
            self.on_retry(k)
        return ready

    def next_wakeup(self) -> float | None:
        return min(self.due.values()) - self.clock() if self.due else None


class IndexedStore:
    """Objects by key, with a secondary index by parent key."""

    def __init__(self, key_of: Callable[[Any], Hashable], parent_of: Callable[[Any], Hashable]):
        self.key_of, self.parent_of = key_of, parent_of
        self.objects: dict = {}

    def apply(self, event) -> set:
        """Apply one event; returns the parent keys whose object sets changed."""
        touched: set = set()
        if isinstance(event, Replace):
            new = {self.key_of(o): o for o in event.objects}
            for k in set(self.objects) | set(new):
                a, b = self.objects.get(k), new.get(k)
                if a != b:
                    touched.update(self.parent_of(x) for x in (a, b) if x is not None)
            self.objects = new
        elif isinstance(event, Upsert):
            k = self.key_of(event.obj)
            old = self.objects.get(k)
            if old != event.obj:
                touched.add(self.parent_of(event.obj))
                if old is not None:
                    touched.add(self.parent_of(old))
                self.objects[k] = event.obj
        elif isinstance(event, Delete):
            old = self.objects.pop(event.key, None)
            if old is not None:
                touched.add(self.parent_of(old))
        else:
            raise TypeError(f"unknown event {event!r}")
        return touched

    def by_parent(self, parent) -> list:
        return [o for o in self.objects.values() if self.parent_of(o) == parent]

    def parents(self) -> set:
        return {self.parent_of(o) for o in self.objects.values()}


class ReconcileLoop:
    def __init__(self, source: Callable[[], AsyncIterator], reconcile: Callable[[Hashable], Awaitable[None]], *,
                 key_of=lambda o: o["key"], parent_of=lambda o: o["parent"], resync_period: float | None = 600.0,
                 failure_base_delay: float = 1.0, failure_max_delay: float = 60.0, source_retry_delay: float = 1.0):
        self.source, self.reconcile = source, reconcile
        self.store = IndexedStore(key_of, parent_of)
        self.queue = WorkQueue()
        self.retry = RetryScheduler(self.queue.add, failure_base_delay, failure_max_delay)
        self.resync_period, self.source_retry_delay = resync_period, source_retry_delay
        self.synced = asyncio.Event()
        self.tasks: list[asyncio.Task] = []
        self.stats = {"reconciled": 0, "failed": 0, "source_restarts": 0}

    async def start(self):
        self.tasks = [asyncio.ensure_future(self._drive_source())]
        await self.synced.wait()                         # the first Replace has been applied
        self.tasks.append(asyncio.ensure_future(self._work()))
        self.tasks.append(asyncio.ensure_future(self._timers()))

    async def stop(self):
        self.queue.shutdown()
        for t in self.tasks:
            t.cancel()
        await asyncio.gather(*self.tasks, return_exceptions=True)
        self.tasks = []

    async def __aenter__(self):
        await self.start()
        return self

    async def __aexit__(self, *exc):
        await self.stop()

    async def _drive_source(self):
        while True:
            try:
                first = True
                async for ev in self.source():
                    assert not first or isinstance(ev, Replace), "a source stream opens with the whole world"
                    first = False
                    for p in sorted(self.store.apply(ev), key=repr):
                        self.queue.add(p)
                    self.synced.set()
            except asyncio.CancelledError:
                raise
            except Exception:
                pass
            self.stats["source_restarts"] += 1
            await asyncio.sleep(self.source_retry_delay)

    async def _work(self):
        while True:
            key = await self.queue.get()
            if key is None:
                return
            try:
                await self.reconcile(key)
                self.retry.note_success(key)
                self.stats["reconciled"] += 1
            except asyncio.CancelledError:
                raise
            except Exception:
                self.stats["failed"] += 1
                self.retry.note_failure(key)

    async def _timers(self):
        last_resync = time.monotonic()
        while True:
            wake = self.retry.next_wakeup()
            await asyncio.sleep(max(0.01, min(wake if wake is not None else 0.25, 0.25)))
            self.retry.release_due()
            if self.resync_period is not None and time.monotonic() - last_resync >= self.resync_period:
                last_resync = time.monotonic()
                for p in self.store.parents():
                    self.queue.add(p)


class LookAgain(Exception):
    """Raised by a reconcile handler that changed the cell it was called for (restarted it, say): the observation is not
    recorded as handled, so the next poll reconciles the cell's new state."""


class PollingReconcileLoop:
    """Lists cells every `interval` seconds and reconciles those whose description changed (None = disappeared).  The
    first listing is reconciled before `start` returns and its failure is raised; later failures are retried next poll."""

    def __init__(self, list_cells: Callable[[], Awaitable[dict]], interval: float = 2.0):
        self.list_cells, self.interval = list_cells, interval
        self.seen: dict = {}
        self.task: asyncio.Task | None = None

    async def poll_once(self, reconcile) -> None:
        observed = await self.list_cells()
        first_error = None
        for cid in sorted(set(self.seen) | set(observed)):
            info = observed.get(cid)
            if self.seen.get(cid) == info:
                continue
            try:
                await reconcile(cid, info)
            except LookAgain:       # the handler acted on the cell: what was observed is already out of date
                continue
            except Exception as e:  # the other cells still get their turn
                first_error = first_error or e
                continue
            if info is None:
                self.seen.pop(cid, None)
            else:
                self.seen[cid] = info
        if first_error is not None:
            raise first_error

    async def start(self, reconcile):
        await self.poll_once(reconcile)

        async def watch():
            while True:
                await asyncio.sleep(self.interval)
                try:
                    await self.poll_once(reconcile)
                except asyncio.CancelledError:
                    raise
                except Exception:
                    pass

        self.task = asyncio.ensure_future(watch())
        return self.stop

    async def stop(self):
        if self.task is not None:
            self.task.cancel()
            await asyncio.gather(self.task, return_exceptions=True)
            self.task = None
