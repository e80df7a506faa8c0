"""Standalone model runner for debugging: forward / backward on given tokens and log-prob comparison against a second
source (another checkpoint, a dumped rollout, or the rollout engine).

Reference: miles/utils/debug_utils/* (`run_megatron` CLI: standalone fwd/bwd + logprob compare, thread dumps, replay of
reward functions).

    python -m miles_b200.utils.debug run --model-name tiny --fp32 --tokens 5,9,13,21 [--hf-checkpoint DIR] [--backward]
    python -m miles_b200.utils.debug compare --model-name tiny --fp32 --rollout-dump dump.pt [--hf-checkpoint DIR]
    python -m miles_b200.utils.debug stacks          # dump the python stack of every thread of THIS process (SIGUSR1 hook)
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import signal
import sys

import torch


def install_stack_dump(sig=signal.SIGUSR1):
    """`kill -USR1 <pid>` prints every thread's python stack to stderr (the in-repo substitute for py-spy dumps)."""
    faulthandler.register(sig, all_threads=True, chain=False)


def _build(a):
    from ..models.config import PRESETS
    from ..models.qwen3 import build_model
    from ..parallel.state import ParallelState

    cfg = PRESETS[a.model_name]
    dev = "cuda" if torch.cuda.is_available() and not a.cpu else "cpu"
    dtype = torch.float32 if a.fp32 or dev == "cpu" else torch.bfloat16
    model = build_model(cfg, ParallelState.single(), dtype=dtype, device=dev, seed=a.seed)
    if a.hf_checkpoint:
        from ..checkpoint import hf_io
        from ..models.convert import load_named_into_model

        load_named_into_model(model, hf_io.load_hf_dir(a.hf_checkpoint).items(), cfg, model.ps)
    return cfg, model, dev


def token_logprobs(model, tokens: list[int], temperature: float = 1.0) -> torch.Tensor:
    """log p(tokens[t+1] | tokens[:t+1]) for t = 0 … n−2."""
    from ..models.qwen3 import ForwardMeta

    dev = next(model.parameters()).device
    T = len(tokens)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32, device=dev),
                       cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=dev), max_seqlen=T)
    h = model(torch.tensor(tokens, dtype=torch.int32, device=dev), meta)
    lp, _ = model.log_probs(h[:-1], torch.tensor(tokens[1:], dtype=torch.int64, device=dev), temperature)
    return lp.float()


def cmd_run(a) -> dict:
    cfg, model, dev = _build(a)
    tokens = [int(t) for t in a.tokens.split(",")]
    with torch.set_grad_enabled(a.backward):
        lp = token_logprobs(model, tokens)
        out = {"tokens": tokens, "logprobs": lp.tolist(), "sum": float(lp.sum())}
        if a.backward:
            (-lp.sum()).backward()
            sq = sum(float(p.grad.float().pow(2).sum()) for p in model.parameters() if p.grad is not None)
            out["grad_norm"] = sq ** 0.5
    return out


def cmd_compare(a) -> dict:
    """Per-sample max |Δ logp| between this model and the log-probs stored in a rollout dump
    (`--save-debug-rollout-data` files)."""
    cfg, model, dev = _build(a)
    raw = torch.load(a.rollout_dump, weights_only=False)
    worst, rows = 0.0, []
    with torch.no_grad():
        for group in raw["samples"][: a.limit]:
            for s in group:
                toks, R = s["tokens"], s["response_length"]
                if not s.get("rollout_log_probs") or R == 0:
                    continue
                lp = token_logprobs(model, toks, a.temperature)[-R:]
                d = (lp.cpu() - torch.tensor(s["rollout_log_probs"])).abs().max().item()
                rows.append({"index": s.get("index"), "max_abs_diff": d})
                worst = max(worst, d)
    return {"max_abs_diff": worst, "samples": rows}


def main(argv=None):
    p = argparse.ArgumentParser(prog="miles_b200.utils.debug")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("run", "compare"):
        s = sub.add_parser(name)
        s.add_argument("--model-name", required=True)
        s.add_argument("--hf-checkpoint", default=None)
        s.add_argument("--fp32", action="store_true")
        s.add_argument("--cpu", action="store_true")
        s.add_argument("--seed", type=int, default=0)
        if name == "run":
            s.add_argument("--tokens", required=True)
            s.add_argument("--backward", action="store_true")
        else:
            s.add_argument("--rollout-dump", required=True)
            s.add_argument("--temperature", type=float, default=1.0)
            s.add_argument("--limit", type=int, default=8)
    sub.add_parser("stacks")
    a = p.parse_args(argv)
    if a.cmd == "stacks":
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        return {}
    out = cmd_run(a) if a.cmd == "run" else cmd_compare(a)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
