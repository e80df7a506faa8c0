"""Audit trail: JSONL event log, analyzer rules, and data witnesses.

Reference: miles/utils/audit_utils/* — an `EventLogger` every component writes structured events to (one JSON object
per line, per process), an analyzer that replays the logs against rules (weight checksums equal between trainer and
engines for every published version; checksums equal across data-parallel replicas after every optimizer step; every
rollout sample consumed by training exactly once), and `_DataWitness`, a tag that travels with each sample through
rollout → conversion → DP split → micro-batching so the analyzer can prove the last rule.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import threading
import time
from collections import Counter, defaultdict
from typing import Any, Iterable

import torch


class EventLogger:
    def __init__(self, directory: str | None, source: str = "main", rank: int = 0):
        self.path = None
        self.source, self.rank = source, rank
        self._lock = threading.Lock()
        self.events: list[dict] = []           # kept in memory too (tests, in-process analysis)
        if directory:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, f"events_{source}_rank{rank}.jsonl")

    def log(self, kind: str, **fields) -> dict:
        ev = {"t": time.time(), "source": self.source, "rank": self.rank, "kind": kind, **fields}
        with self._lock:
            self.events.append(ev)
            if self.path:
                with open(self.path, "a") as f:
                    f.write(json.dumps(ev, default=str) + "\n")
        return ev


def read_events(directory: str) -> list[dict]:
    out = []
    for p in sorted(glob.glob(os.path.join(directory, "events_*.jsonl"))):
        with open(p) as f:
            out += [json.loads(line) for line in f if line.strip()]
    out.sort(key=lambda e: e["t"])
    return out


# ---- checksums ---------------------------------------------------------------------------------------------------

def tensor_checksum(t: torch.Tensor) -> str:
    """Order-sensitive digest of the raw bytes (bit-exact equality test, not a norm)."""
    b = t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()
    return hashlib.blake2b(b, digest_size=8).hexdigest()


def model_checksums(named: Iterable[tuple[str, torch.Tensor]]) -> dict[str, str]:
    return {n: tensor_checksum(t) for n, t in named}


def combined_checksum(checks: dict[str, str]) -> str:
    h = hashlib.blake2b(digest_size=8)
    for n in sorted(checks):
        h.update(n.encode())
        h.update(checks[n].encode())
    return h.hexdigest()


# ---- witnesses -----------------------------------------------------------------------------------------------------

class DataWitness:
    """Allocates witness ids for rollout samples and records where they are consumed."""

    def __init__(self, logger: EventLogger):
        self.logger = logger
        self._next = 0

    def allocate(self, rollout_id: int, n: int, namespace: int = 0) -> list[int]:
        """`namespace` keeps ids of allocators that run side by side apart (one per rollout rank when every rank trains on
        what it generated)."""
        base = (int(namespace) << 40) + self._next
        ids = list(range(base, base + n))
        self._next += n
        self.logger.log("witness_allocated", rollout_id=rollout_id, ids=ids)
        return ids

    def consumed(self, rollout_id: int, step: int, ids: list[int], dp_rank: int = 0):
        self.logger.log("witness_consumed", rollout_id=rollout_id, step=step, ids=list(ids), dp_rank=dp_rank)


# ---- analyzer ------------------------------------------------------------------------------------------------------

class Finding(dict):
    pass


def rule_weight_checksums(events: list[dict]) -> list[Finding]:
    """For every weight version, each engine's checksum equals the trainer's."""
    trainer: dict[int, str] = {}
    out = []
    for e in events:
        if e["kind"] == "weights_published":
            trainer[e["version"]] = e["checksum"]
    for e in events:
        if e["kind"] == "weights_received":
            want = trainer.get(e["version"])
            if want is None:
                out.append(Finding(rule="weight_checksums", problem="engine received an unpublished version", event=e))
            elif want != e["checksum"]:
                out.append(Finding(rule="weight_checksums", problem="engine weights differ from trainer", version=e["version"],
                                   engine=e.get("engine"), want=want, got=e["checksum"]))
    return out


def rule_cross_replica(events: list[dict]) -> list[Finding]:
    """After every optimizer step all data-parallel replicas hold identical parameters."""
    by_step: dict[int, dict[Any, str]] = defaultdict(dict)
    for e in events:
        if e["kind"] == "replica_checksum":
            by_step[e["step"]][e.get("dp_rank", e["rank"])] = e["checksum"]
    return [Finding(rule="cross_replica", problem="replicas diverged", step=s, checksums=dict(c))
            for s, c in sorted(by_step.items()) if len(set(c.values())) > 1]


def rule_witness(events: list[dict]) -> list[Finding]:
    """Every allocated sample is consumed exactly once (per optimizer pass over its rollout)."""
    alloc: dict[int, int] = {}
    used: Counter = Counter()
    for e in events:
        if e["kind"] == "witness_allocated":
            for i in e["ids"]:
                alloc[i] = e["rollout_id"]
        elif e["kind"] == "witness_consumed":
            used.update(e["ids"])
    out = []
    missing = [i for i in alloc if used[i] == 0]
    dup = [i for i, c in used.items() if c > 1]
    unknown = [i for i in used if i not in alloc]
    if missing:
        out.append(Finding(rule="witness", problem="samples never trained on", ids=missing[:20], count=len(missing)))
    if dup:
        out.append(Finding(rule="witness", problem="samples trained on more than once", ids=dup[:20], count=len(dup)))
    if unknown:
        out.append(Finding(rule="witness", problem="consumed ids that were never allocated", ids=unknown[:20]))
    return out


RULES = {"weight_checksums": rule_weight_checksums, "cross_replica": rule_cross_replica, "witness": rule_witness}


def analyze(events_or_dir, rules: list[str] | None = None) -> list[Finding]:
    events = read_events(events_or_dir) if isinstance(events_or_dir, str) else list(events_or_dir)
    out: list[Finding] = []
    for name in rules or list(RULES):
        out += RULES[name](events)
    return out


def main():
    import argparse

    p = argparse.ArgumentParser(description="replay audit logs against the rules")
    p.add_argument("directory")
    p.add_argument("--rules", nargs="*", default=None, choices=sorted(RULES))
    a = p.parse_args()
    findings = analyze(a.directory, a.rules)
    for f in findings:
        print(json.dumps(f, default=str))
    raise SystemExit(1 if findings else 0)


if __name__ == "__main__":
    main()
