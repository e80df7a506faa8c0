"""Headline benchmark: GRPO tokens/s per box (rollout + log-prob + train + weight sync), Qwen3-30B-A3B shape.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run, one rank per GPU)
    python bench.py --impl reference ...                     (the unmodified reference, if it can run here)

One step = the public-API GRPO step of this package on synthetic data:
    rollout (colocated engine, token-in-token-out, paged KV, sampling with log-probs and routed experts)
    → rule reward (1 if last generated id mod 7 == 0) → group-normalised advantages
    → trainer forward-only log-probs → GRPO forward/backward over packed micro-batches → distributed Adam
    → weight hand-over to the engine.
Weak scaling: 8 prompts × 8 samples and 16 experts per GPU, expert-parallel over all N GPUs; at N = 8 this is exactly
the named config (64 prompts × 8 samples, 128 experts, top-8).  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_T_PROCESS_START = time.time()
BASELINE_TOKENS_PER_S = None  # the reference publishes no GRPO tokens/s figure for this config


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--model", default="qwen3-30B-A3B")
    p.add_argument("--layers", type=int, default=None, help="override the layer count (development only; marks the run invalid)")
    p.add_argument("--prompts-per-gpu", type=int, default=8)
    p.add_argument("--samples-per-prompt", type=int, default=8)
    p.add_argument("--prompt-len-min", type=int, default=256)
    p.add_argument("--prompt-len-max", type=int, default=2048)
    p.add_argument("--max-new-tokens", type=int, default=8192)
    p.add_argument("--mean-response-len", type=int, default=512,
                   help="stop-token set sized so that a random-init policy stops after this many tokens on average")
    p.add_argument("--max-tokens-per-gpu", type=int, default=32768, help="token budget of a micro-batch (the reference recipe's value)")
    p.add_argument("--mem-fraction-static", type=float, default=0.75,
                   help="share of device memory for weights + optimizer state + KV cache; the rest (45 GB at 0.75) stays free for "
                        "training activations. Too small a KV cache caps how many of the 64 requests decode at once.")
    p.add_argument("--no-fused", action="store_true", help="NCCL + separate GEMM baseline instead of the fused kernels")
    p.add_argument("--no-cuda-graph", action="store_true")
    p.add_argument("--fp8-recipe", choices=["none", "mxfp8"], default="none",
                   help="mxfp8: forward projections (dense and expert) on the block-scaled tensor-core path, backward in bf16 — the "
                        "secondary MXFP8 training config; the headline run is bf16")
    p.add_argument("--warmup-max-new-tokens", type=int, default=256,
                   help="response cap of the untimed warm-up steps (same pipeline, same prompts and batch: graphs, allocator pools, "
                        "communicators and clocks are warmed by the prompt-dominated work; the cap keeps 5 warm-up steps of the "
                        "8-GPU run inside a fixed launch window); 0 = the full cap")
    p.add_argument("--deadline-seconds", type=float, default=830.0,
                   help="wall-clock budget of this process: when the next timed step is projected to end after it, the timed loop stops "
                        "and the line reports the steps actually timed (`steps` < `steps_requested`, `stopped_early` set) instead of being "
                        "lost with the process; 0 = no deadline")
    p.add_argument("--no-weight-sync-probe", action="store_true",
                   help="skip the untimed measurement of a weight sync into an engine that holds its own copy of the weights")
    p.add_argument("--quiet", action="store_true")
    return p.parse_args()


def reference_arm(a):
    """The reference needs ray, megatron.core, sglang and sglang_router, none of which is installed or in the offline
    wheelhouse; `pip install --no-deps` of the reference itself succeeds but `miles.utils.arguments` cannot be imported."""
    why = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import miles  # noqa: F401
        for mod in ("ray", "megatron.core", "sglang"):
            try:
                __import__(mod)
            except Exception as e:
                why = f"reference installed with --no-deps but its runtime stack is missing: import {mod} failed ({type(e).__name__})"
                break
    except Exception as e:
        why = f"reference package not importable from baseline/_ref ({type(e).__name__}: {e})"
    if why is None:
        why = "reference stack importable but no offline model/data path is wired; not run"
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def _weight_sync_probe(args, cfg, ps, actor, dev, world):
    """After the timed region: the trainer's weights into an engine that holds ITS OWN copy (the timed loop's engine serves the
    trainer's parameters directly, so its hand-over is a version bump).  Pause → every bucket copied into the engine's buffers
    by the one-kernel NVLink / device copy → resume, three times after one warm-up; device time, maximum over ranks."""
    import torch
    import torch.distributed as dist

    try:
        from miles_b200.engine.engine import Engine
        from miles_b200.weight_update.updater import WeightUpdater

        other = Engine(cfg, model=None, ps=ps, device=dev, dtype=torch.bfloat16, num_blocks=8, max_running_requests=8,
                       max_context_len=512, seed=99, use_cuda_graph=False)
        upd = WeightUpdater(args, actor, [other], mode="nvlink")
        info = upd.update_weights()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(3):
            info = upd.update_weights()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 3e3, (time.perf_counter() - t0) / 3], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        a_, b_ = next(iter(actor.model.parameters())), next(iter(other.model.parameters()))
        return {"seconds": float(t[0]), "seconds_wall": float(t[1]), "bytes_per_gpu": int(info.get("bytes", 0)),
                "identical_after_sync": bool(torch.equal(a_.data, b_.data)), "mode": "nvlink (one kernel per bucket into the engine's own buffers)"}
    except Exception as e:          # the probe must never cost the run its result line
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm(a)

    import torch
    import torch.distributed as dist

    from miles_b200.args import parse_args
    from miles_b200.models.config import get_config
    from miles_b200.ops import cuda as K
    from miles_b200.orchestration.rollout_executor import RolloutExecutor
    from miles_b200.orchestration.wiring import update_weights
    from miles_b200.parallel.state import ParallelState, init_distributed
    from miles_b200.rollout.client import InProcEngineClient
    from miles_b200.rollout.data_source import SyntheticPromptSource
    from miles_b200.train.actor import TrainActor
    from miles_b200.utils import object_store
    from miles_b200.weight_update.updater import WeightUpdater

    rank, world, local = init_distributed()
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run for N > 1)"
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)

    base = get_config(a.model)
    experts = base.num_experts if world >= 8 else max(base.moe_topk, 16 * world)
    cfg = base.with_(num_experts=experts, num_layers=a.layers or base.num_layers)
    full_config = (experts == base.num_experts and a.layers is None)

    if world > 1:
        ps = ParallelState.build(tp=1, ep=world, sequence_parallel=False)
        ps.fused = not a.no_fused
        if ps.fused:
            from miles_b200.parallel.fabric import Fabric

            try:
                ps.fabric = Fabric.create(ps)
                # dispatch / return buffers are sized from the largest micro-batch (or prefill batch) a rank can see
                ps.fabric.moe_max_tokens = max(a.max_tokens_per_gpu, 16384) + 2048
            except Exception as e:      # peer mapping refused on this box: run the NCCL path and say so in `fused_comm`
                print(f"[bench] fabric unavailable ({type(e).__name__}: {e}); falling back to NCCL collectives", file=sys.stderr)
                ps.fused, ps.fabric = False, None
    else:
        ps = ParallelState.single()

    V = cfg.vocab_size
    # stop-token set: a random-init policy is close to uniform over the vocabulary, so |stop set| / V ≈ 1 / mean length
    n_stop = max(1, V // max(1, a.mean_response_len))
    stop_ids = list(range(V - n_stop, V))
    gb = a.prompts_per_gpu * world
    argv = (f"--rollout-batch-size {gb} --n-samples-per-prompt {a.samples_per_prompt} "
            f"--rollout-max-response-len {a.max_new_tokens} --num-rollout 1000000 --rm-type last_mod7 --lr 1e-6 --colocate "
            f"--advantage-estimator grpo --eps-clip 0.2 --use-dynamic-batch-size --max-tokens-per-gpu {a.max_tokens_per_gpu} "
            f"--recompute-granularity full --use-rollout-routing-replay --balance-data "
            f"--expert-model-parallel-size {world} --rollout-temperature 1.0 --rollout-data-exchange local"
            + (" --fp8-recipe mxfp8" if a.fp8_recipe == "mxfp8" else ""))
    args = parse_args(argv.split())
    args.rollout_stop_token_ids = stop_ids

    actor = TrainActor(args, ps, device=dev)
    actor.init(cfg)

    from miles_b200.engine.engine import Engine

    engine = Engine(cfg, model=actor.model, ps=ps, device=dev, dtype=torch.bfloat16, mem_fraction_static=a.mem_fraction_static,
                    max_running_requests=a.prompts_per_gpu * a.samples_per_prompt, max_prefill_tokens=16384,
                    max_context_len=a.prompt_len_max + a.max_new_tokens, seed=1234 + rank, use_cuda_graph=not a.no_cuda_graph)
    if rank == 0 and not a.quiet:
        print(f"[engine] KV cache: {engine.allocator.num_free} blocks x {engine.block_size} tokens = "
              f"{engine.allocator.num_free * engine.block_size} tokens", file=sys.stderr, flush=True)
    client = InProcEngineClient([engine])
    source = SyntheticPromptSource(args, V - n_stop, a.prompt_len_min, a.prompt_len_max, seed=1000 + rank)
    executor = RolloutExecutor(args, source, client, ps=ps, rollout_dp_size=world, rollout_dp_rank=rank)
    updater = WeightUpdater(args, actor, [engine])

    class Rollout:
        engines = [engine]

    Rollout.executor = executor
    phases: dict = {}
    counters = {"tokens": 0, "gen_tokens": 0, "h2d": 0, "d2h": 0, "sync_s": 0.0, "rollout_s": 0.0, "train_s": 0.0}
    from miles_b200.train import data as train_data

    stall_s = int(os.environ.get("MILES_STALL_DUMP_S", "0"))

    def step(i):
        if stall_s:   # dump every thread's python stack and exit if one step takes longer than this
            import faulthandler

            faulthandler.dump_traceback_later(stall_s, exit=True)
        try:
            return _step(i)
        finally:
            if stall_s:
                import faulthandler

                faulthandler.cancel_dump_traceback_later()

    def _step(i):
        t0 = time.perf_counter()
        pack = executor.get(i)
        t1 = time.perf_counter()
        shard = object_store.get(pack.data_ref)
        metrics = actor.train(i, shard)
        object_store.remove(pack.data_ref)
        t2 = time.perf_counter()
        info = update_weights(args, actor, Rollout, updater)
        t3 = time.perf_counter()
        counters["tokens"] += int(pack.metrics["rollout/total_tokens"])
        counters["gen_tokens"] += int(pack.metrics.get("rollout/response_tokens", 0))
        counters["rollout_s"] += t1 - t0
        counters["train_s"] += t2 - t1
        counters["sync_s"] += t3 - t2
        # counted where the copies are made: the engine's prefill inputs, per-decode-step row state and sampled ids /
        # log-probs / routed experts (pinned buffers of the decode runner); the trainer's packed micro-batches (pinned
        # staging, `train/data.to_device`); the loss metrics read back at the end of the step
        counters["h2d"] += engine.stats.get("h2d_bytes", 0) + train_data.TRANSFER["h2d_bytes"]
        counters["d2h"] += engine.stats.get("d2h_bytes", 0) + 4 * len(metrics)
        engine.stats["h2d_bytes"] = engine.stats["d2h_bytes"] = 0
        train_data.TRANSFER["h2d_bytes"] = 0
        counters["engine"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in engine.stats.items()}
        for k, v in metrics.items():                       # the trainer's own phase timers (seconds, this rank)
            if k.startswith("perf/") and k.endswith("_time"):
                phases[k[5:-5]] = phases.get(k[5:-5], 0.0) + float(v)
        return metrics

    full_cap = args.rollout_max_response_len
    warm_cap = min(full_cap, a.warmup_max_new_tokens) if a.warmup_max_new_tokens > 0 else full_cap
    for i in range(a.warmup):
        args.rollout_max_response_len = executor.local_args.rollout_max_response_len = warm_cap
        try:
            m = step(i)
        finally:
            args.rollout_max_response_len = executor.local_args.rollout_max_response_len = full_cap
        if rank == 0 and not a.quiet:
            print(f"[warmup {i}] tokens={counters['tokens']} rollout={counters['rollout_s']:.1f}s train={counters['train_s']:.1f}s "
                  f"loss={m.get('train/loss', float('nan')):.4g} grad_norm={m.get('train/grad_norm', float('nan')):.4g}",
                  file=sys.stderr, flush=True)
    for k in counters:
        counters[k] = 0
    phases.clear()
    for k in list(engine.stats):
        engine.stats[k] = type(engine.stats[k])()
    launches0 = K.launch_count()
    sampler = ClockSampler(local)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    ev0.record()
    steps_done = 0
    for i in range(a.steps):
        if i > 0 and a.deadline_seconds > 0:
            # every rank takes the decision of rank 0 (one tiny all-reduce per step)
            el = time.perf_counter() - wall0
            late = torch.tensor([float((time.time() - _T_PROCESS_START) + 1.05 * el / i > a.deadline_seconds) if rank == 0 else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(late, op=dist.ReduceOp.MAX)
            if float(late) > 0:
                break
        step(a.warmup + i)
        steps_done = i + 1
        if rank == 0 and not a.quiet:
            # progress on stderr (host clock, this rank): what a reader has if the run is stopped before the JSON line
            el = time.perf_counter() - wall0
            print(f"[step {i + 1}/{a.steps}] elapsed={el:.1f}s s/step={el / (i + 1):.2f} tokens={counters['tokens']} "
                  f"tokens/s={counters['tokens'] / el:.0f} rollout={counters['rollout_s']:.1f}s train={counters['train_s']:.1f}s",
                  file=sys.stderr, flush=True)
    ev1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    dev_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else {}
    launches = K.launch_count() - launches0
    t = torch.tensor([dev_ms, wall * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    # executor.get gathers all ranks' samples, so `tokens` already counts the whole job
    total_tokens = counters["tokens"]
    gen_tokens = counters["gen_tokens"]
    err = K.check_error_flag()
    if a.no_weight_sync_probe:
        sync_probe = None
    elif world >= 8:
        # the 8-GPU run has no seconds to spare inside its launch window; the per-GPU copy is the one measured at N = 1, 2, 4
        sync_probe = {"skipped": "not run at 8 GPUs (same per-GPU copy as at fewer GPUs; see the 1- and 2-GPU lines)"}
    else:
        sync_probe = _weight_sync_probe(args, cfg, ps, actor, dev, world)
    if rank == 0:
        value = total_tokens / (dev_ms / 1e3)
        out = {
            "metric": "GRPO tokens/s/box (rollout+train+weight-sync)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": steps_done, "steps_requested": a.steps, "stopped_early": (None if steps_done == a.steps else f"deadline of {a.deadline_seconds:.0f} s for the whole process: {steps_done} of {a.steps} steps timed"), "warmup": a.warmup, "warmup_max_new_tokens": warm_cap, "ms_per_step": dev_ms / steps_done, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16" if a.fp8_recipe == "none" else "mxfp8 forward (e4m3, 1x32 e8m0 scales) + bf16 backward",
            "data": "synthetic prompts (uniform random ids), random-init weights, rule reward (last id mod 7 == 0)",
            "config": {
                "model": f"{cfg.name}-shaped MoE: {cfg.num_layers} layers, hidden {cfg.hidden_size}, {cfg.num_heads}q/{cfg.num_kv_heads}kv "
                         f"heads, {cfg.num_experts} experts top-{cfg.moe_topk}, expert FFN {cfg.moe_ffn_hidden_size}, vocab {V}",
                "named_config": bool(full_config),
                "note": None if full_config else "16 experts per GPU (expert-parallel weak scaling): the 128-expert model with "
                        "Adam state needs ~490 GB and only fits at 8 GPUs; active parameters per token are identical",
                "global_batch": gb * a.samples_per_prompt, "prompts": gb, "samples_per_prompt": a.samples_per_prompt,
                "prompt_len": [a.prompt_len_min, a.prompt_len_max], "max_new_tokens": a.max_new_tokens,
                "mean_response_len_target": a.mean_response_len, "seq_len": a.prompt_len_max + a.max_new_tokens,
                "parallelism": f"ep{world}-dp{world}", "fused_comm": bool(ps.fabric is not None),
                "cache": "inputs larger than L2 (weights + KV + activations ≫ 126 MB per step)",
                "warmup_steps": ("same pipeline, prompts and batch as the timed steps"
                                 + (f", responses capped at {warm_cap} new tokens" if warm_cap != full_cap else ", full response cap")),
            },
            "clocks": clocks,
            "e2e": {"value": total_tokens / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": counters["h2d"] // steps_done,
                    "d2h_bytes_per_step": counters["d2h"] // steps_done, "timed": "wall clock around the public-API step "
                    "(RolloutExecutor.get → TrainActor.train → update_weights), max over ranks"},
            "gpu_launches": int(launches),
            "breakdown_s_per_step": {"rollout": counters["rollout_s"] / steps_done, "train": counters["train_s"] / steps_done,
                                     "weight_sync": counters["sync_s"] / steps_done},
            "train_phases_s_per_step_rank0": {k: round(v / steps_done, 3) for k, v in sorted(phases.items())},
            "tokens_per_step": total_tokens // steps_done, "kernel_error_flag": err, "weight_sync_own_copy": sync_probe,
            # the reference's perf/tokens_per_gpu_per_sec counts response tokens only: the same quantity for the whole job
            "generated_tokens_per_s": gen_tokens / (dev_ms / 1e3), "generated_tokens_per_step": gen_tokens // steps_done,
            "engine_stats_rank0": counters.get("engine"),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
