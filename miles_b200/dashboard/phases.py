"""Per-rank phase intervals: who did what when.

Every `Timer` span of a trainer rank (log_probs, actor_train, update_weights, …) and every rollout of the executor is written
as one JSON line `{rank, role, phase, start, end, rollout_id}` under `<dump>/dashboard/phases.rank<r>.jsonl`; the viewer draws
them as lanes, and the advisories look for gaps.  Writing is append-only and never raises into the training path
(reference: miles/dashboard/hooks.py:63-160 `PhaseSink`, collector.py).
"""
from __future__ import annotations

import glob
import json
import os
import time


class PhaseSink:
    def __init__(self, directory: str, rank: int, role: str = "trainer"):
        self.path = os.path.join(directory, "dashboard", f"phases.rank{rank}.jsonl")
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        self.rank, self.role = rank, role
        self.rollout_id = -1
        # Timer reports (name, duration) at the END of a span with a monotonic clock: intervals are rebuilt on the wall clock
        self._skew = time.time() - time.perf_counter()

    def __call__(self, name: str, dt: float):
        end = time.perf_counter() + self._skew
        self.write(name, end - dt, end)

    def write(self, phase: str, start: float, end: float, **extra):
        try:
            with open(self.path, "a") as f:
                f.write(json.dumps({"rank": self.rank, "role": self.role, "phase": phase, "start": start, "end": end,
                                    "rollout_id": self.rollout_id, **extra}) + "\n")
        except OSError:
            pass                                   # a full disk must not stop training


def read_phases(directory: str) -> list[dict]:
    rows = []
    for p in sorted(glob.glob(os.path.join(directory, "dashboard", "phases.rank*.jsonl"))):
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line:
                    try:
                        rows.append(json.loads(line))
                    except ValueError:
                        pass                       # a line still being written
    rows.sort(key=lambda r: (r["start"], r["rank"]))
    return rows


def lanes(rows: list[dict]) -> dict[str, list[dict]]:
    out: dict[str, list[dict]] = {}
    for r in rows:
        out.setdefault(f"{r['role']}:{r['rank']}", []).append(r)
    return out


def utilisation(rows: list[dict]) -> dict:
    """Share of the run's wall time every lane spent in each phase, and its idle share (time covered by no top-level span).
    Nested spans (a phase inside another) count once, through the union of intervals."""
    if not rows:
        return {}
    t0, t1 = min(r["start"] for r in rows), max(r["end"] for r in rows)
    wall = max(t1 - t0, 1e-9)
    out = {}
    for lane, rs in lanes(rows).items():
        by_phase: dict[str, float] = {}
        for r in rs:
            by_phase[r["phase"]] = by_phase.get(r["phase"], 0.0) + (r["end"] - r["start"])
        busy, cur_s, cur_e = 0.0, None, None
        for r in sorted(rs, key=lambda r: r["start"]):
            if cur_e is None or r["start"] > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                cur_s, cur_e = r["start"], r["end"]
            else:
                cur_e = max(cur_e, r["end"])
        if cur_e is not None:
            busy += cur_e - cur_s
        out[lane] = {"phases": {k: v / wall for k, v in sorted(by_phase.items())}, "idle": max(0.0, 1.0 - busy / wall), "wall_s": wall}
    return out


def gaps(rows: list[dict], min_gap_s: float = 30.0) -> list[dict]:
    """Stretches of at least `min_gap_s` in which a lane recorded nothing (a stall, a hang, a very slow collective)."""
    found = []
    for lane, rs in lanes(rows).items():
        rs = sorted(rs, key=lambda r: r["start"])
        end = rs[0]["end"]
        for r in rs[1:]:
            if r["start"] - end >= min_gap_s:
                found.append({"lane": lane, "start": end, "end": r["start"], "seconds": r["start"] - end, "before": r["phase"]})
            end = max(end, r["end"])
    return found
