"""Micro-benchmark of one engine decode step (device-timed with CUDA events).

    python -m miles_b200.engine.bench_decode --model qwen3-30B-A3B --experts 16 --batch 64 --context 1536 [--layers N]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m miles_b200.engine.bench_decode --batch 8 --layers 12

Reports the CUDA-graph replay time of the decode step, the eager time of the same step, and the host-side time of
`Engine.step()` around it, so that launch-bound, bandwidth-bound and host-bound shares can be told apart.  Under torchrun
the experts are sharded over the ranks (`--experts` per rank) and the step runs through the fused dispatch/combine
kernels in lockstep; `--kernel-table` adds the per-kernel device time of a step (CUPTI activity records of four steps:
shares only, the step time itself is measured without the tracer; `MILES_PDL=0` gives durations free of dependency waits).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="qwen3-30B-A3B")
    p.add_argument("--experts", type=int, default=16)
    p.add_argument("--layers", type=int, default=None)
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--context", type=int, default=1536)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--record-routing", action="store_true")
    p.add_argument("--kernel-table", action="store_true", help="per-kernel device time of a step (torch.profiler, shares only)")
    p.add_argument("--no-fused", action="store_true", help="expert parallelism through NCCL all-to-all instead of the fabric kernels")
    a = p.parse_args()

    import os

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import get_config
    from miles_b200.parallel.state import ParallelState, init_distributed

    rank, world, local = init_distributed() if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1, 0)
    cfg = get_config(a.model)
    if cfg.is_moe:
        cfg = cfg.with_(num_experts=a.experts * world)
    if a.layers:
        cfg = cfg.with_(num_layers=a.layers)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    ps = None
    if world > 1:
        ps = ParallelState.build(tp=1, ep=world, sequence_parallel=False)
        ps.fused = not a.no_fused
        if ps.fused:
            from miles_b200.parallel.fabric import Fabric

            ps.fabric = Fabric.create(ps)
    eng = Engine(cfg, ps=ps, device=dev, dtype=torch.bfloat16, max_running_requests=a.batch,
                 max_context_len=a.context + 8 * a.steps + 128, mem_fraction_static=0.5, seed=0)
    if world > 1:
        return _lockstep(a, eng, cfg, rank, world)
    g = torch.Generator().manual_seed(0)
    reqs = []
    for i in range(a.batch):
        ids = torch.randint(3, cfg.vocab_size, (a.context,), generator=g).tolist()
        reqs.append(eng.add_request(ids, {"temperature": 1.0, "max_new_tokens": 4 * a.steps + 32}, return_routed_experts=a.record_routing))
    while eng.waiting:
        eng.step()                      # prefill
    torch.cuda.synchronize()
    for _ in range(3):
        eng.step()                      # warm-up + graph capture
    torch.cuda.synchronize()
    runner = eng.runner
    out = {"model": cfg.name, "layers": cfg.num_layers, "experts": cfg.num_experts, "batch": a.batch, "context": a.context}
    # host + device, as the engine runs it
    t0 = time.perf_counter()
    for _ in range(a.steps):
        eng.step()
    torch.cuda.synchronize()
    out["engine_step_ms"] = (time.perf_counter() - t0) * 1e3 / a.steps
    # graph replay only
    key = next(iter(runner.graphs)) if runner.graphs else None
    if key is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            runner.graphs[key].replay()
        e1.record()
        torch.cuda.synchronize()
        out["graph_replay_ms"] = e0.elapsed_time(e1) / a.steps
        out["launches_in_graph"] = runner.launches_per_graph[key]
        B, record = key
        e0.record()
        for _ in range(a.steps):
            runner._forward(B, record)
        e1.record()
        torch.cuda.synchronize()
        out["eager_ms"] = e0.elapsed_time(e1) / a.steps
    if a.kernel_table:
        _kernel_table(eng, out)
    print(json.dumps(out))


def _kernel_table(eng, out, steps: int = 4):
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            eng.step()
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total / steps, e.count / steps) for e in prof.key_averages() if e.device_time_total > 0]
    rows.sort(key=lambda r: -r[1])
    out["kernel_table_us_per_step"] = [{"kernel": k[:90], "us": round(t, 1), "launches": round(c, 1)} for k, t, c in rows[:24]]


def _lockstep(a, eng, cfg, rank, world):
    """Expert-parallel ranks: every step is a collective, so all ranks run the same number of steps."""
    import torch.distributed as dist

    g = torch.Generator().manual_seed(rank)
    n_steps = 12 + a.steps + (4 if a.kernel_table else 0)
    for _ in range(a.batch):
        ids = torch.randint(3, cfg.vocab_size, (a.context,), generator=g).tolist()
        eng.add_request(ids, {"temperature": 1.0, "max_new_tokens": 2 * n_steps + 64}, return_routed_experts=a.record_routing)
    eng.begin_rollout()
    for _ in range(12):
        eng.step()                      # prefill(s), warm-up, graph capture
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        eng.step()
    torch.cuda.synchronize()
    ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / a.steps], device=eng.device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"model": cfg.name, "layers": cfg.num_layers, "experts": cfg.num_experts, "ep": world, "batch_per_rank": a.batch,
           "context": a.context, "fused_comm": bool(eng.ps.fabric is not None), "engine_step_ms_max_over_ranks": float(ms),
           "launches_in_graph": next(iter(eng.runner.launches_per_graph.values()), None)}
    if a.kernel_table:
        _kernel_table(eng, out)
    if rank == 0:
        print(json.dumps(out))
    eng.abort_request(None)
    eng.finish_rollout()
    while not eng.global_done:
        eng.step()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
