"""Process groups that can be torn down and rebuilt while the job keeps running.

An NCCL communicator pins device memory for its buffers and channels.  When a colocated trainer sleeps so that the
rollout engine can use the GPU, the trainer's communicators are dead weight; the reference wraps every group so that
all of them can be destroyed on `sleep` and re-created (same ranks, same options, same order on every rank) on
`wake_up` (miles/utils/reloadable_process_group.py:15-315, used by miles/backends/megatron_utils/actor.py:455,495,507,897).

Here nothing is monkey-patched: groups are made through a registry that remembers how each was made and WHO HOLDS the
handle (object, attribute).  `destroy_all()` destroys the communicators and clears the holders' attributes — a
collective issued on a released group fails loudly with "group is None" rather than using a dangling handle —
`reload_all()` re-creates them in creation order and re-points every holder.  The default (world) group stays.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field
from typing import Any

import torch.distributed as dist


@dataclass
class _Entry:
    ranks: list[int]
    kwargs: dict
    handle: Any = None
    holders: list = field(default_factory=list)        # (weakref to object, attribute)


class GroupRegistry:
    def __init__(self):
        self.entries: list[_Entry] = []
        self.released = False
        self.stats = {"destroyed": 0, "reloaded": 0}

    def new_group(self, ranks: list[int], **kwargs):
        """`dist.new_group` (collective over the world, as usual) recorded for later reloads."""
        handle = dist.new_group(list(ranks), **kwargs)
        self.entries.append(_Entry(list(ranks), dict(kwargs), handle))
        return handle

    def _entry_of(self, handle) -> _Entry | None:
        return next((e for e in self.entries if e.handle is handle and handle is not None), None)

    def bind(self, obj, attr: str) -> bool:
        """Declare that `obj.attr` holds a handle made by this registry; it will follow reloads."""
        e = self._entry_of(getattr(obj, attr, None))
        if e is None:
            return False
        e.holders.append((weakref.ref(obj), attr))
        return True

    def destroy_all(self) -> int:
        """Collective in effect (every rank must do the same): destroy every recorded group, clear the holders."""
        n = 0
        for e in self.entries:
            if e.handle is None:
                continue
            if dist.get_rank() in e.ranks:
                try:
                    dist.destroy_process_group(e.handle)
                except Exception:
                    pass                                   # already invalid: nothing left to free
            for ref, attr in e.holders:
                o = ref()
                if o is not None:
                    setattr(o, attr, None)
            e.handle = None
            n += 1
        self.released = True
        self.stats["destroyed"] += n
        return n

    def reload_all(self) -> int:
        """Collective: re-create every destroyed group in creation order and re-point the holders."""
        n = 0
        for e in self.entries:
            if e.handle is not None:
                continue
            e.handle = dist.new_group(e.ranks, **e.kwargs)
            member = dist.get_rank() in e.ranks
            for ref, attr in e.holders:
                o = ref()
                if o is not None:
                    setattr(o, attr, e.handle if member else None)
            n += 1
        self.released = False
        self.stats["reloaded"] += n
        return n


REGISTRY = GroupRegistry()
