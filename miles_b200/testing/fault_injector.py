"""Host-side fault injection for fault-tolerance tests.

The reference ships a fault injector and FT test actions with its package (miles/utils/test_utils/*,
`TrainRayActor` fault-injection RPCs, miles/ray/train_actor.py:56-243).  This one acts on the host only, at points
where the process has no kernel or collective in flight: it raises an exception, exits the process, sleeps (a slow
rank), drops a message, or substitutes an error code for a call's result.  It never touches the device.

Rules come from code (`inject(...)`) or from the environment:

    MILES_FAULT_INJECT="rank=1,step=3,point=before_allreduce,kind=raise;rank=0,step=5,kind=exit"
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass


class InjectedFault(RuntimeError):
    """Raised by `kind=raise` rules."""


@dataclass
class Rule:
    kind: str                       # raise | exit | sleep | drop | error_code
    rank: int | None = None
    step: int | None = None
    point: str | None = None
    arg: float = 0.0                # sleep seconds / error code
    once: bool = True
    fired: int = 0

    def matches(self, rank: int, step: int | None, point: str | None) -> bool:
        if self.once and self.fired:
            return False
        return ((self.rank is None or self.rank == rank) and (self.step is None or self.step == step)
                and (self.point is None or self.point == point))


class FaultInjector:
    def __init__(self, rank: int | None = None, rules: list[Rule] | None = None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.rules = list(rules or [])
        env = os.environ.get("MILES_FAULT_INJECT")
        if env:
            self.rules += parse_rules(env)
        self.log: list[tuple] = []

    def inject(self, kind: str, **kw) -> Rule:
        r = Rule(kind=kind, **kw)
        self.rules.append(r)
        return r

    def at(self, point: str, step: int | None = None):
        """Call at a named host-side point (between steps / before a collective is issued)."""
        for r in self.rules:
            if r.kind in ("drop", "error_code") or not r.matches(self.rank, step, point):
                continue
            r.fired += 1
            self.log.append((r.kind, point, step))
            if r.kind == "raise":
                raise InjectedFault(f"injected fault at {point} (rank {self.rank}, step {step})")
            if r.kind == "exit":
                os._exit(int(r.arg) or 17)
            if r.kind == "sleep":
                time.sleep(r.arg)

    def should_drop(self, point: str, step: int | None = None) -> bool:
        """True when a message passing through `point` must be discarded (the caller simply does not send it)."""
        for r in self.rules:
            if r.kind == "drop" and r.matches(self.rank, step, point):
                r.fired += 1
                self.log.append(("drop", point, step))
                return True
        return False

    def error_code(self, point: str, default: int = 0, step: int | None = None) -> int:
        """Result code of a call that a test wants to see fail (a fake of the failing call, not a real failure)."""
        for r in self.rules:
            if r.kind == "error_code" and r.matches(self.rank, step, point):
                r.fired += 1
                self.log.append(("error_code", point, step))
                return int(r.arg)
        return default


def parse_rules(spec: str) -> list[Rule]:
    rules = []
    for part in spec.split(";"):
        part = part.strip()
        if not part:
            continue
        kv = dict(x.split("=", 1) for x in part.split(","))
        rules.append(Rule(kind=kv.get("kind", "raise"), rank=int(kv["rank"]) if "rank" in kv else None,
                          step=int(kv["step"]) if "step" in kv else None, point=kv.get("point"),
                          arg=float(kv.get("arg", 0.0)), once=kv.get("once", "1") != "0"))
    return rules


GLOBAL = FaultInjector()          # the process-wide injector: product code calls `GLOBAL.at(point)` at a few host-side points


def arm(point: str, error: BaseException | None = None, step: int | None = None) -> Rule:
    """Make the next pass through `point` in this process raise (used by the cell API's inject-fault)."""
    return GLOBAL.inject("raise", point=point, step=step, rank=GLOBAL.rank)
