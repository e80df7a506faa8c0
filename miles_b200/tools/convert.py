"""Checkpoint converters (one CLI, sub-commands), counterparts of the reference's `tools/*.py`:

    python -m miles_b200.tools.convert hf-to-torch-dist  --hf DIR --out DIR [--model-name NAME]
    python -m miles_b200.tools.convert torch-dist-to-hf  --load DIR --out DIR --hf-config DIR|--model-name NAME
    python -m miles_b200.tools.convert hf-to-fp8         --hf DIR --out DIR        (128×128 block e4m3 + weight_scale_inv)
    python -m miles_b200.tools.convert hf-to-mxfp8       --hf DIR --out DIR        (1×32 block e4m3 + ue8m0 scales)
    python -m miles_b200.tools.convert hf-to-nvfp4       --hf DIR --out DIR [--four-over-six] [--all-linears] [--ignore …]   (packed e2m1 + scales)
    python -m miles_b200.tools.convert hf-to-int4        --hf DIR --out DIR [--group-size 32] [--asymmetric]                 (compressed-tensors)
    python -m miles_b200.tools.convert hf-to-nvfp4-qdq   --hf DIR --out DIR        (bf16 values that went through NVFP4)
    python -m miles_b200.tools.convert hf-to-int4-qdq    --hf DIR --out DIR [--block 1 32] [--asymmetric]
    python -m miles_b200.tools.convert fp8-to-bf16       --hf DIR --out DIR        (dequantise block-scaled FP8 weights)

(reference: tools/convert_hf_to_torch_dist.py, convert_torch_dist_to_hf.py, convert_hf_to_fp8.py, convert_hf_to_mxfp8.py,
convert_hf_to_nvfp4.py, convert_hf_to_int4.py, fp8_cast_bf16.py:16 `weight_dequant_kernel`).  Tensors are processed
one safetensors shard at a time; quantisation kernels run on the GPU when one is present, else through the fp32
reference implementations.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil

import torch

from .. import ops
from ..checkpoint import hf_io, torch_dist
from ..models import convert as mc
from ..models.config import PRESETS, ModelConfig
from ..weight_update.quantize import hf_quant_config, quantize_hf_tensors, should_quantize


def _cfg(args) -> ModelConfig:
    d = getattr(args, "hf_config", None) or getattr(args, "hf", None)
    if d and os.path.exists(os.path.join(d, "config.json")):
        with open(os.path.join(d, "config.json")) as f:
            return ModelConfig.from_hf_config(json.load(f))
    assert getattr(args, "model_name", None), "need --model-name or a directory with config.json"
    return PRESETS[args.model_name]


def _dev():
    return "cuda" if torch.cuda.is_available() else "cpu"


def _copy_aux(src: str, dst: str, config_update: dict | None = None):
    """Tokenizer / generation config files travel unchanged; config.json gains the quantisation block."""
    os.makedirs(dst, exist_ok=True)
    for f in os.listdir(src):
        if f.endswith((".json", ".txt", ".model", ".jinja")) and not f.endswith(".safetensors.index.json") and f != "config.json":
            shutil.copy(os.path.join(src, f), os.path.join(dst, f))
    cp = os.path.join(src, "config.json")
    if os.path.exists(cp):
        with open(cp) as f:
            cfg = json.load(f)
        cfg.update(config_update or {})
        with open(os.path.join(dst, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)


def _shards(hf_dir: str):
    files = sorted(f for f in os.listdir(hf_dir) if f.endswith(".safetensors"))
    assert files, f"no safetensors under {hf_dir}"
    for f in files:
        yield f, hf_io.load_safetensors(os.path.join(hf_dir, f))


def _write_index(out: str, weight_map: dict[str, str], total: int):
    with open(os.path.join(out, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)


def _map_shards(args, fn, config_update=None):
    os.makedirs(args.out, exist_ok=True)
    wm, total = {}, 0
    for fname, tensors in _shards(args.hf):
        out = dict(fn(list(tensors.items())))
        hf_io.save_safetensors(os.path.join(args.out, fname), out, {"format": "pt"})
        for n, t in out.items():
            wm[n] = fname
            total += t.numel() * t.element_size()
    _write_index(args.out, wm, total)
    _copy_aux(args.hf, args.out, config_update)
    return wm


# ---- sub-commands ------------------------------------------------------------------------------------------------

def hf_to_torch_dist(args):
    cfg = _cfg(args)
    ours = mc.hf_state_to_ours(hf_io.load_hf_dir(args.hf), cfg)
    d = torch_dist.save_state(mc.ours_to_megatron(ours, cfg), args.out, iteration=None)
    with open(os.path.join(args.out, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("release")
    rel = os.path.join(args.out, "release")
    if d != rel:
        os.makedirs(rel, exist_ok=True)
        for f in os.listdir(args.out):
            if f.endswith(".distcp") or f == ".metadata":
                shutil.move(os.path.join(args.out, f), os.path.join(rel, f))
    return rel


def torch_dist_to_hf(args):
    cfg = _cfg(args)
    ours = mc.megatron_to_ours(torch_dist.load_state(args.load), cfg)
    named = [x for n, t in ours.items() for x in mc.to_hf(n, t, cfg)]
    hf_io.save_hf_sharded(args.out, [named], cfg, write=True, src_dir=getattr(args, "hf_config", None))
    return args.out


def hf_to_quant(args, mode: str):
    dev = _dev()

    def fn(named):
        named = [(n, t.to(dev) if should_quantize(n, t) else t) for n, t in named]
        return [(n, t.cpu()) for n, t in quantize_hf_tensors(named, mode)]

    return _map_shards(args, fn, hf_quant_config(mode))


def hf_to_packed(args, mode: str):
    """Packed NVFP4 (ModelOpt layout) / compressed-tensors int4 export of an HF directory."""
    from ..weight_update import quant_export as qe

    dev = _dev()
    if mode == "nvfp4":
        opts = dict(ignore=args.ignore, four_over_six=args.four_over_six, all_linears=args.all_linears, pair_strict=False)
        cfg = qe.quant_config("nvfp4", ignore=args.ignore, four_over_six=args.four_over_six)
    else:
        opts = dict(ignore=args.ignore, group_size=args.group_size, symmetric=not args.asymmetric)
        cfg = qe.quant_config("int4", group_size=args.group_size, symmetric=not args.asymmetric, ignore=args.ignore)

    def fn(named):
        named = [(n, t.to(dev) if t.dim() == 2 else t) for n, t in named]
        return [(n, t.cpu()) for n, t in quantize_hf_tensors(named, mode, **opts)]

    return _map_shards(args, fn, cfg)


def hf_to_nvfp4_qdq(args):
    dev = _dev()

    def fn(named):
        out = []
        for n, t in named:
            if should_quantize(n, t) and t.shape[-1] % 16 == 0:
                out.append((n, ops.nvfp4_qdq(t.to(dev).bfloat16()).cpu().to(t.dtype)))
            else:
                out.append((n, t))
        return out

    return _map_shards(args, fn, {"quantization_config": {"quant_method": "nvfp4_qdq", "group_size": 16}})


def hf_to_int4_qdq(args):
    dev = _dev()
    bm, bn = args.block

    def fn(named):
        out = []
        for n, t in named:
            if should_quantize(n, t) and t.shape[0] % bm == 0 and t.shape[1] % bn == 0:
                y, _ = ops.int4_fake_quant(t.to(dev).bfloat16(), bm, bn, not args.asymmetric)
                out.append((n, y.cpu().to(t.dtype)))
            else:
                out.append((n, t))
        return out

    return _map_shards(args, fn, {"quantization_config": {"quant_method": "int4_qdq", "block": [bm, bn], "symmetric": not args.asymmetric}})


def fp8_to_bf16(args):
    def fn(named):
        d = dict(named)
        out = []
        for n, t in named:
            if n.endswith("_scale_inv"):
                continue
            s = d.get(n + "_scale_inv")
            if s is None:
                out.append((n, t))
            elif s.dtype == torch.uint8:
                out.append((n, ops.mxfp8_dequant(t, s).reshape(t.shape).bfloat16()))
            else:
                out.append((n, ops.fp8_blockwise_dequant(t, s).bfloat16()))
        return out

    wm = _map_shards(args, fn, None)
    cp = os.path.join(args.out, "config.json")
    if os.path.exists(cp):
        with open(cp) as f:
            cfg = json.load(f)
        cfg.pop("quantization_config", None)
        with open(cp, "w") as f:
            json.dump(cfg, f, indent=1)
    return wm


def main(argv=None):
    p = argparse.ArgumentParser(prog="miles_b200.tools.convert")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("hf-to-torch-dist", "hf-to-fp8", "hf-to-mxfp8", "hf-to-nvfp4-qdq", "hf-to-int4-qdq", "fp8-to-bf16"):
        s = sub.add_parser(name)
        s.add_argument("--hf", required=True)
        s.add_argument("--out", required=True)
        s.add_argument("--model-name", default=None)
        if name == "hf-to-int4-qdq":
            s.add_argument("--block", type=int, nargs=2, default=[1, 32])
            s.add_argument("--asymmetric", action="store_true")
    for name in ("hf-to-nvfp4", "hf-to-int4"):
        s = sub.add_parser(name)
        s.add_argument("--hf", required=True)
        s.add_argument("--out", required=True)
        s.add_argument("--model-name", default=None)
        s.add_argument("--ignore", nargs="*", default=[])
        if name == "hf-to-nvfp4":
            s.add_argument("--four-over-six", action="store_true")
            s.add_argument("--all-linears", action="store_true")
        else:
            s.add_argument("--group-size", type=int, default=32)
            s.add_argument("--asymmetric", action="store_true")
    s = sub.add_parser("torch-dist-to-hf")
    s.add_argument("--load", required=True)
    s.add_argument("--out", required=True)
    s.add_argument("--hf-config", default=None)
    s.add_argument("--model-name", default=None)
    a = p.parse_args(argv)
    return {"hf-to-torch-dist": hf_to_torch_dist, "torch-dist-to-hf": torch_dist_to_hf,
            "hf-to-fp8": lambda x: hf_to_quant(x, "fp8"), "hf-to-mxfp8": lambda x: hf_to_quant(x, "mxfp8"),
            "hf-to-nvfp4": lambda x: hf_to_packed(x, "nvfp4"), "hf-to-int4": lambda x: hf_to_packed(x, "int4"),
            "hf-to-nvfp4-qdq": hf_to_nvfp4_qdq, "hf-to-int4-qdq": hf_to_int4_qdq, "fp8-to-bf16": fp8_to_bf16}[a.cmd](a)


if __name__ == "__main__":
    main()
