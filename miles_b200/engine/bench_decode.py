"""Micro-benchmark of one engine decode step (device-timed with CUDA events).

    python -m miles_b200.engine.bench_decode --model qwen3-30B-A3B --experts 16 --batch 64 --context 1536 [--layers N]

Reports the CUDA-graph replay time of the decode step, the eager time of the same step, and the host-side time of
`Engine.step()` around it, so that launch-bound, bandwidth-bound and host-bound shares can be told apart.
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
    a = p.parse_args()

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import get_config

    cfg = get_config(a.model)
    if cfg.is_moe:
        cfg = cfg.with_(num_experts=a.experts)
    if a.layers:
        cfg = cfg.with_(num_layers=a.layers)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    eng = Engine(cfg, device=dev, dtype=torch.bfloat16, max_running_requests=a.batch, max_context_len=a.context + 4 * a.steps + 64,
                 mem_fraction_static=0.5, seed=0)
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
    print(json.dumps(out))


if __name__ == "__main__":
    main()
