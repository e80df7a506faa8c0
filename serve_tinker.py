"""Tinker-compatible multi-LoRA training gateway.

    python serve_tinker.py --model-name qwen3-0.6B --hf-checkpoint DIR --lora-rank 32 --lora-num-slots 8 --tinker-port 8000

Counterpart of the reference's `serve_tinker.py` (serve_tinker.py:27-96): builds the base model with adapter slots, an
engine that aliases it for sampling, and serves the Tinker API (`miles_b200/tinker/server.py`) with uvicorn.
"""
from __future__ import annotations

import torch

from miles_b200.args import build_parser, validate_args


def build_service(args):
    from miles_b200.args import model_config_from_args
    from miles_b200.engine.engine import Engine
    from miles_b200.models.qwen3 import build_model
    from miles_b200.parallel.state import ParallelState
    from miles_b200.tinker.service import TinkerService
    from miles_b200.train import lora

    cfg = model_config_from_args(args)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    dtype = torch.float32 if getattr(args, "fp32", False) or device == "cpu" else torch.bfloat16
    ps = ParallelState.single()
    model = build_model(cfg, ps, dtype=dtype, device=device, seed=args.seed)
    hf = getattr(args, "hf_checkpoint", None)
    if hf:
        from miles_b200.checkpoint import hf_io
        from miles_b200.models.convert import load_named_into_model

        load_named_into_model(model, hf_io.load_hf_dir(hf).items(), cfg, ps)
    assert args.lora_rank > 0, "--lora-rank is required for the tinker gateway"
    lora.apply_lora(model, args)
    ek = dict(getattr(args, "engine_kwargs", {}) or {})
    engine = Engine(cfg, model=model, ps=ps, device=device, dtype=dtype, num_blocks=ek.get("num_blocks"),
                    block_size=ek.get("block_size"), use_cuda_graph=False, seed=args.rollout_seed)
    return TinkerService(model, args, engine=engine, pad_multiple=128 if device == "cuda" else 1)


def serve(argv=None):
    import uvicorn

    from miles_b200.args import _split_engine_args
    from miles_b200.tinker.server import build_app

    p = build_parser()
    p.add_argument("--tinker-host", default="127.0.0.1")
    p.add_argument("--tinker-port", type=int, default=8000)
    import sys

    rest, engine_kwargs = _split_engine_args(list(sys.argv[1:] if argv is None else argv))
    args = p.parse_args(rest)
    args.engine_kwargs = engine_kwargs
    args.num_rollout = args.num_rollout or 0
    validate_args(args)
    uvicorn.run(build_app(build_service(args)), host=args.tinker_host, port=args.tinker_port, log_level="info")


if __name__ == "__main__":
    serve()
