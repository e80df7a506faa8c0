"""RolloutExecutor: run the rollout function, convert samples to train data, split by DP.

Reference: miles/ray/rollout/rollout_executor.py:53-338 (get / eval / save / load /
set_weight_version) and train_data_conversion.py.  Process model here is SPMD: every rank owns a
rollout-DP slice of the prompt groups (its engine, or its TP/EP group of engines, generates them);
the slices are exchanged with one object all-gather so every rank sees the same global batch, which
is then partitioned over the trainer's data-parallel ranks.
"""
from __future__ import annotations

import json
import os
import pickle
import time
from typing import Any

import torch
import torch.distributed as dist

from ..rollout.inference_rollout import InferenceRolloutFn, RolloutFnEvalInput, RolloutFnTrainInput
from ..train.data import convert_samples_to_train_data, split_train_data_by_dp
from ..types import RolloutDataPack, Sample
from ..utils import object_store
from ..utils.misc import load_function


_FOREIGN_ID_STRIDE = 1 << 40


def plan_group_moves(sizes: list[list[int]], max_moves: int = 256) -> list[tuple[int, int, int]]:
    """Which prompt groups change ranks so that the token counts even out: `sizes[r][i]` = tokens of rank r's group i →
    [(source rank, group index on the source, destination rank)].  Greedy: the fullest rank gives the emptiest one the
    group closest to half their difference, as long as a group smaller than the difference exists (every move then lowers
    the pair's maximum).  Groups move at most once; deterministic, so every rank computes the same plan."""
    loads = [sum(s) for s in sizes]
    avail = [{i: n for i, n in enumerate(s)} for s in sizes]           # groups still at home
    moves = []
    while len(moves) < max_moves and len(loads) > 1:
        hi = max(range(len(loads)), key=lambda r: (loads[r], -r))
        lo = min(range(len(loads)), key=lambda r: (loads[r], r))
        gap = loads[hi] - loads[lo]
        cand = [(abs(n - gap / 2), i) for i, n in avail[hi].items() if 0 < n < gap]
        if not cand:
            break
        _, i = min(cand)
        n = avail[hi].pop(i)
        loads[hi] -= n
        loads[lo] += n
        moves.append((hi, i, lo))
    return moves


class RolloutExecutor:
    def __init__(self, args, data_source, client, *, ps=None, rollout_dp_size: int = 1, rollout_dp_rank: int = 0,
                 gather_group=None, eval_sources=None, tracker=None):
        self.args, self.data_source, self.client = args, data_source, client
        self.ps = ps
        self.rollout_dp_size, self.rollout_dp_rank = rollout_dp_size, rollout_dp_rank
        self.gather_group = gather_group
        self.tracker = tracker
        self.weight_version = 0
        path = getattr(args, "rollout_function_path", None)
        fn_cls = load_function(path) if path else InferenceRolloutFn
        self.local_args = self._localise(args)
        self.rollout_fn = fn_cls(self.local_args, data_source, client, eval_sources) if isinstance(fn_cls, type) else fn_cls
        self.eval_fn = self.rollout_fn
        if getattr(args, "eval_function_path", None):
            ef = load_function(args.eval_function_path)
            self.eval_fn = ef(self.local_args, data_source, client, eval_sources) if isinstance(ef, type) else ef

    def _localise(self, args):
        """Each rollout-DP rank produces its share of the rollout batch."""
        import copy

        a = copy.copy(args)
        if self.rollout_dp_size > 1:
            assert args.rollout_batch_size % self.rollout_dp_size == 0, "rollout_batch_size must divide rollout DP"
            a.rollout_batch_size = args.rollout_batch_size // self.rollout_dp_size
            a.over_sampling_batch_size = max(1, (args.over_sampling_batch_size or args.rollout_batch_size) // self.rollout_dp_size)
        return a

    # ---------------------------------------------------------------------------------------
    def get(self, rollout_id: int) -> RolloutDataPack:
        args = self.args
        t0 = time.time()
        if getattr(args, "load_debug_rollout_data", None):
            path = args.load_debug_rollout_data.format(rollout_id=rollout_id)
            raw = torch.load(path, weights_only=False)
            groups = [[Sample.from_dict(d) for d in g] for g in raw["samples"]]
            metrics = {}
        else:
            out = self._call(self.rollout_fn, RolloutFnTrainInput(rollout_id))
            groups, metrics = out.samples, dict(out.metrics)
        dp = self.ps.dp_size if self.ps is not None else 1
        # one engine per data-parallel rank: the rank may keep what it generated (prompt groups are never split, so group
        # normalisation is unaffected) instead of pickling every sample — routed experts included — to every rank
        mode = getattr(args, "rollout_data_exchange", "gather")
        local = (mode in ("local", "balanced") and self.rollout_dp_size > 1
                 and dp == self.rollout_dp_size and dist.is_initialized() and self._is_rollout_leader())
        t_gen = time.time() - t0
        if not local:
            groups = self._exchange(groups)
        elif mode == "balanced":
            groups = self._rebalance(groups)
        if getattr(args, "save_debug_rollout_data", None) and (not dist.is_initialized() or dist.get_rank() == 0):
            path = args.save_debug_rollout_data.format(rollout_id=rollout_id)
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
            torch.save({"rollout_id": rollout_id, "samples": [[s.to_dict() for s in g] for g in groups]}, path)
        post = getattr(args, "rollout_all_samples_process_path", None)
        if post:
            load_function(post)(args, groups)
        witness = getattr(self, "witness", None)
        if witness is None and getattr(args, "audit_dir", None):
            from ..audit.events import DataWitness, EventLogger

            rank = dist.get_rank() if dist.is_initialized() else 0
            witness = self.witness = DataWitness(EventLogger(args.audit_dir, "rollout", rank))
        data = convert_samples_to_train_data(args, groups)
        if witness is not None:
            # every sample of the batch gets an id here and the trainer reports the ids it consumed: the audit analyser
            # then proves that no sample was dropped or trained on twice
            data["witness_ids"] = witness.allocate(rollout_id, len(data["tokens"]), namespace=self.rollout_dp_rank if local else 0)
        if getattr(args, "rollout_data_postprocess_path", None):
            load_function(args.rollout_data_postprocess_path)(args, data)
        metrics.update(self._rollout_metrics(groups, data, time.time() - t0))
        metrics["perf/generate_time"] = t_gen
        if getattr(args, "use_miles_dashboard", False) and getattr(args, "dump_details", None):
            from ..dashboard.phases import PhaseSink

            sink = getattr(self, "_phase_sink", None)
            if sink is None:
                sink = self._phase_sink = PhaseSink(args.dump_details, dist.get_rank() if dist.is_initialized() else 0, "rollout")
            sink.rollout_id = rollout_id
            sink.write("generate", t0, t0 + t_gen)
            sink.write("rollout", t0, time.time())
        if local:
            metrics = self._reduce_metrics(metrics, len(data["tokens"]), sum(data["response_lengths"]))
            shard = dict(data)
            shard["partition"] = list(range(len(data["tokens"])))
        else:
            shards = split_train_data_by_dp(args, data, dp)
            shard = shards[self.ps.dp_rank if self.ps is not None else 0]
        ref = object_store.put(shard)
        return RolloutDataPack(rollout_id=rollout_id, sample_indices=data["sample_indices"], data_ref=ref, metrics=metrics)

    def eval(self, rollout_id: int) -> dict:
        out = self._call(self.eval_fn, RolloutFnEvalInput(rollout_id))
        metrics = {}
        for name, d in out.data.items():
            r = d["rewards"]
            metrics[f"eval/{name}"] = sum(r) / max(1, len(r))
            metrics[f"eval/{name}-truncated_ratio"] = sum(d["truncated"]) / max(1, len(r))
        if self.tracker is not None:
            self.tracker.log(metrics, step=rollout_id, step_key="eval/step")
        return metrics

    def _call(self, fn, inp):
        return fn(inp)

    def _exchange(self, groups: list[list[Sample]]) -> list[list[Sample]]:
        if self.rollout_dp_size <= 1 or not dist.is_initialized():
            return groups
        from ..utils import ragged_codec

        world = dist.get_world_size(self.gather_group)
        # per-token fields travel as flat typed arrays with offsets (one buffer per field), not as lists of Python numbers
        payload = ragged_codec.encode_groups(groups) if self._is_rollout_leader() else None
        gathered: list = [None] * world
        dist.all_gather_object(gathered, payload, group=self.gather_group)
        out = []
        for part in gathered:
            if part:
                out.extend(ragged_codec.decode_groups(part, Sample))
        out.sort(key=lambda g: g[0].index if g[0].index is not None else 0)
        return out

    def _rebalance(self, groups: list[list[Sample]]) -> list[list[Sample]]:
        """Local exchange with the token counts evened out: ranks agree on a plan from the per-group token counts (a few
        integers per rank), then only the groups that move travel, point to point, as ragged-codec buffers."""
        from ..utils import ragged_codec

        g = self.gather_group if self.gather_group is not None else dist.group.WORLD
        world, me = dist.get_world_size(g), dist.get_rank(g)
        sizes = [sum(len(s.tokens) for s in grp) for grp in groups]
        all_sizes: list = [None] * world
        dist.all_gather_object(all_sizes, sizes, group=g)
        moves = plan_group_moves(all_sizes)
        if not moves:
            return groups
        dev = "cuda" if dist.get_backend(g) == "nccl" else "cpu"
        out_blobs = {}
        for src, idx, dst in moves:
            if src == me:
                blob = pickle.dumps(ragged_codec.encode_groups([groups[idx]]), protocol=5)
                out_blobs[(idx, dst)] = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
        lens: list = [None] * world
        dist.all_gather_object(lens, {k: int(v.numel()) for k, v in out_blobs.items()}, group=g)
        ops, recv = [], []
        for src, idx, dst in moves:                                    # the same order on every rank
            if src == me:
                ops.append(dist.P2POp(dist.isend, out_blobs[(idx, dst)].to(dev), dist.get_global_rank(g, dst), group=g))
            elif dst == me:
                buf = torch.empty(lens[src][(idx, dst)], dtype=torch.uint8, device=dev)
                recv.append((src, buf))
                ops.append(dist.P2POp(dist.irecv, buf, dist.get_global_rank(g, src), group=g))
        for w in (dist.batch_isend_irecv(ops) if ops else []):
            w.wait()
        gone = {idx for src, idx, _ in moves if src == me}
        kept = [grp for i, grp in enumerate(groups) if i not in gone]
        for src, buf in recv:
            for grp in ragged_codec.decode_groups(pickle.loads(buf.cpu().numpy().tobytes()), Sample):
                # every rank numbers its own samples: keep the newcomers' ids apart from this rank's (rows with one
                # rollout id are treated as segments of one rollout downstream)
                for smp in grp:
                    if smp.index is not None:
                        smp.index += (src + 1) * _FOREIGN_ID_STRIDE
                    if isinstance(smp.rollout_id, int):
                        smp.rollout_id += (src + 1) * _FOREIGN_ID_STRIDE
                kept.append(grp)
        return kept

    def _reduce_metrics(self, m: dict, n_samples: int, n_resp: int) -> dict:
        """Whole-job values of the per-rank rollout metrics (local exchange mode): means are re-weighted by their own
        denominators (samples, or response tokens for the log-prob mean), totals summed, extrema reduced."""
        by_sample = ["rollout/raw_reward", "rollout/response_len/mean", "rollout/truncated_ratio"]
        dev = "cuda" if dist.get_backend(self.gather_group) == "nccl" else "cpu"
        sums = torch.tensor([float(n_samples), float(n_resp), m.get("rollout/total_tokens", 0.0),
                             m.get("rollout/log_probs", 0.0) * n_resp] + [m.get(k, 0.0) * n_samples for k in by_sample],
                            dtype=torch.float64, device=dev)
        ext = torch.tensor([m.get("rollout/response_len/max", 0.0), -m.get("rollout/response_len/min", 0.0),
                            m.get("perf/rollout_time", 0.0), m.get("perf/generate_time", 0.0)], dtype=torch.float64, device=dev)
        dist.all_reduce(sums, group=self.gather_group)
        dist.all_reduce(ext, op=dist.ReduceOp.MAX, group=self.gather_group)
        sums, ext = sums.tolist(), ext.tolist()
        n, r = max(sums[0], 1.0), max(sums[1], 1.0)
        out = dict(m)
        out["rollout/total_tokens"] = sums[2]
        out["rollout/response_tokens"] = sums[1]
        if "rollout/log_probs" in m:
            out["rollout/log_probs"] = sums[3] / r
        for i, k in enumerate(by_sample):
            out[k] = sums[4 + i] / n
        out["rollout/response_len/max"], out["rollout/response_len/min"] = ext[0], -ext[1]
        out["perf/rollout_time"], out["perf/generate_time"] = ext[2], ext[3]
        gpus = max(1, getattr(self.args, "rollout_num_gpus", 1) or 1)
        out["perf/tokens_per_gpu_per_sec"] = sums[1] / max(ext[2], 1e-9) / gpus
        return out

    def _is_rollout_leader(self) -> bool:
        # within a TP/EP engine group every rank holds identical samples; one of them contributes
        return getattr(self, "is_leader", True)

    def _rollout_metrics(self, groups, data, dt) -> dict:
        flat = [s for g in groups for s in g]
        if not flat:
            return {}
        resp = [s.response_length for s in flat]
        m = {
            "rollout/raw_reward": sum(data["raw_reward"]) / len(flat),
            "rollout/response_len/mean": sum(resp) / len(resp),
            "rollout/response_len/max": max(resp),
            "rollout/response_len/min": min(resp),
            "rollout/truncated_ratio": sum(data["truncated"]) / len(flat),
            "rollout/total_tokens": float(sum(data["total_lengths"])),
            "rollout/response_tokens": float(sum(resp)),
            "perf/rollout_time": dt,
            "perf/tokens_per_gpu_per_sec": sum(resp) / max(dt, 1e-9) / max(1, getattr(self.args, "rollout_num_gpus", 1) or 1),
        }
        if "rollout_log_probs" in data:
            tot = sum(sum(x) for x in data["rollout_log_probs"])
            m["rollout/log_probs"] = tot / max(1, sum(resp))
        return m

    # ---------------------------------------------------------------------------------------
    def save(self, rollout_id: int):
        self.data_source.save(rollout_id)

    def load(self, rollout_id: int | None):
        self.data_source.load(rollout_id)

    def set_weight_version(self, v: int):
        self.weight_version = v
        if hasattr(self.rollout_fn, "set_weight_version"):      # staleness accounting of the fully-async producer
            self.rollout_fn.set_weight_version(v)

    def shutdown(self):
        if hasattr(self.rollout_fn, "stop"):
            self.rollout_fn.stop()
