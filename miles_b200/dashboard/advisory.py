"""Advisories: what a person reading the dashboard would notice, stated as findings with a hint.

Inputs: the metric series (`SeriesStore`), the phase intervals, the rollout dumps.  Each rule returns zero or more
`Advisory(severity, title, detail, hint)`; none of them changes anything (reference: miles/dashboard/advisory.py:54-400 —
stall, engine-alarm, rollout, data-parallel spread, MFU and tuning advisories).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

from . import phases as ph


@dataclass
class Advisory:
    severity: str            # info | warn | alarm
    title: str
    detail: str
    hint: str = ""


def _last(store, name, n=20):
    return [y for _, y in store.get(name, n)]


def _mean(xs):
    return sum(xs) / len(xs) if xs else None


def stall_advisories(rows: list[dict], min_gap_s: float = 60.0) -> list[Advisory]:
    out = []
    for g in ph.gaps(rows, min_gap_s):
        out.append(Advisory("alarm" if g["seconds"] > 5 * min_gap_s else "warn", f"{g['lane']} recorded nothing for {g['seconds']:.0f} s",
                            f"no phase between {g['start']:.0f} and {g['end']:.0f}; the next one was {g['before']}",
                            "a rank waiting in a collective for a slower or dead peer looks like this: compare the lanes at that time"))
    return out


def spread_advisories(rows: list[dict], phase: str = "actor_train", tolerance: float = 0.15) -> list[Advisory]:
    per_lane: dict[str, float] = {}
    for r in rows:
        if r["phase"] == phase:
            lane = f"{r['role']}:{r['rank']}"
            per_lane[lane] = per_lane.get(lane, 0.0) + r["end"] - r["start"]
    if len(per_lane) < 2:
        return []
    lo, hi = min(per_lane.values()), max(per_lane.values())
    if hi <= 0 or (hi - lo) / hi <= tolerance:
        return []
    slow = max(per_lane, key=per_lane.get)
    return [Advisory("warn", f"{phase} time differs by {(hi - lo) / hi:.0%} across ranks", f"slowest: {slow} ({hi:.1f} s), fastest {lo:.1f} s",
                     "every rank waits for the slowest at the optimizer step: balance the data (--balance-data, gathered exchange) "
                     "or lower --max-tokens-per-gpu so that micro-batches even out")]


def rollout_advisories(store) -> list[Advisory]:
    out = []
    trunc = _mean(_last(store, "rollout/truncated_ratio"))
    if trunc is not None and trunc > 0.2:
        out.append(Advisory("warn", f"{trunc:.0%} of the responses hit the length limit", "truncated samples carry no terminal signal",
                            "raise --rollout-max-response-len, or mask them with --mask-truncated-samples"))
    dropped = _mean(_last(store, "rollout/dynamic_filter_dropped"))
    if dropped is not None and dropped > 0:
        kept = _mean(_last(store, "rollout/response_len/mean"))
        out.append(Advisory("info", f"the dynamic filter drops {dropped:.1f} prompt groups per rollout", f"mean kept response length {kept}",
                            "groups whose samples all score the same teach nothing under GRPO; raise --over-sampling-batch-size if the "
                            "rollout runs short of groups"))
    diff = _mean(_last(store, "train/train_rollout_logprob_abs_diff"))
    if diff is not None and diff > 0.05:
        out.append(Advisory("alarm", f"trainer and engine disagree on log-probs by {diff:.3f} on average",
                            "the policy that sampled is not the policy being trained",
                            "check the weight sync (--check-weight-update-equal), routing replay for MoE models, or run --true-on-policy-mode"))
    return out


def efficiency_advisories(store, rows: list[dict]) -> list[Advisory]:
    out = []
    gen, train = _mean(_last(store, "perf/rollout_time")), _mean(_last(store, "perf/train_time"))
    if gen and train and gen > 2.5 * train:
        out.append(Advisory("info", f"generation takes {gen / (gen + train):.0%} of a step", f"rollout {gen:.1f} s vs train {train:.1f} s",
                            "the tail of long responses runs at tiny batch sizes: partial rollouts / over-sampling, or asynchronous "
                            "training (train_async.py) hide it"))
    mfu = _mean(_last(store, "perf/mfu"))
    if mfu is not None and mfu < 0.15:
        out.append(Advisory("info", f"model FLOP utilisation of the train phase is {mfu:.1%}", "",
                            "larger --max-tokens-per-gpu, less recomputation (--recompute-granularity selective) if memory allows"))
    retr = _mean(_last(store, "engine/retractions"))
    if retr:
        out.append(Advisory("warn", f"the engine retracts {retr:.1f} requests per rollout", "the KV cache is too small for the running batch",
                            "raise --sglang-mem-fraction-static or lower --sglang-max-running-requests"))
    util = ph.utilisation(rows)
    for lane, u in util.items():
        if u["idle"] > 0.5 and u["wall_s"] > 60:
            out.append(Advisory("info", f"{lane} is idle {u['idle']:.0%} of the time", "", "colocated jobs alternate phases by design; "
                                "a disaggregated trainer that idles this much has too few engines feeding it"))
    return out


def compute_advisories(store, rows: list[dict], min_gap_s: float = 60.0) -> list[dict]:
    found = stall_advisories(rows, min_gap_s) + spread_advisories(rows) + rollout_advisories(store) + efficiency_advisories(store, rows)
    order = {"alarm": 0, "warn": 1, "info": 2}
    return [asdict(a) for a in sorted(found, key=lambda a: order[a.severity])]
