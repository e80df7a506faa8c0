"""Hugging Face checkpoint IO: safetensors shards + `model.safetensors.index.json`.

A self-contained reader/writer of the safetensors container (8-byte little-endian header length,
JSON header `{name: {dtype, shape, data_offsets}}`, raw little-endian tensor bytes) so that export
works for every dtype the weight-sync quantisers emit (bf16, fp8 e4m3, uint8 e8m0 scales).  Export
layout follows the reference's snapshot publisher
(miles/backends/training_utils/weight_update/snapshot_publisher.py:61-99, hf_export.py:31-86):
`model-{i:05d}-of-{n:05d}.safetensors`, the index json, copied config/tokenizer files, `.complete`.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
from typing import Iterable, Iterator

import numpy as np
import torch

_DT = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_DT_INV = {v: k for k, v in _DT.items()}


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def save_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None):
    header: dict = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    off = 0
    order = list(tensors)
    for n in order:
        t = tensors[n]
        nb = _nbytes(t)
        header[n] = {"dtype": _DT_INV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nb]}
        off += nb
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((-len(hjson)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for n in order:
            t = tensors[n].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")   # reshape first: a scalar has no last dim to reinterpret
    os.replace(tmp, path)


def read_safetensors_header(path: str) -> tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return header, 8 + n


def load_safetensors(path: str, names: Iterable[str] | None = None) -> dict[str, torch.Tensor]:
    header, base = read_safetensors_header(path)
    want = set(names) if names is not None else None
    out = {}
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    for n, info in header.items():
        if n == "__metadata__" or (want is not None and n not in want):
            continue
        a, b = info["data_offsets"]
        dt = _DT[info["dtype"]]
        buf = torch.from_numpy(np.array(mm[base + a: base + b]))  # copy out of the mapping
        out[n] = buf.view(dt).reshape(info["shape"])
    return out


def load_hf_dir(directory: str, names: Iterable[str] | None = None) -> dict[str, torch.Tensor]:
    idx = os.path.join(directory, "model.safetensors.index.json")
    files: list[str]
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        files = sorted(set(wm.values()))
    else:
        files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    out: dict[str, torch.Tensor] = {}
    for fn in files:
        out.update(load_safetensors(os.path.join(directory, fn), names))
    return out


def save_hf_sharded(directory: str, named_iter: Iterator[list[tuple[str, torch.Tensor]]] | Iterable, cfg, *,
                    write: bool = True, src_dir: str | None = None, max_shard_bytes: int = 5 << 30,
                    extra_config: dict | None = None):
    """Consume buckets of (hf_name, tensor) (every rank must iterate: the iterator runs collectives) and,
    on the writing rank, emit size-bounded shards plus the index."""
    if write:
        os.makedirs(directory, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    total = 0
    for bucket in named_iter:
        items = bucket if isinstance(bucket, list) else [bucket]
        for n, t in items:
            if not write:
                continue
            nb = _nbytes(t)
            if size + nb > max_shard_bytes and shards[-1]:
                shards.append({})
                size = 0
            shards[-1][n] = t.detach().cpu()
            size += nb
            total += nb
    if not write:
        return
    n = len(shards)
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        save_safetensors(os.path.join(directory, fn), sh, {"format": "pt"})
        for k in sh:
            weight_map[k] = fn
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    conf = cfg.to_hf_config()
    if extra_config:
        conf.update(extra_config)
    if src_dir and os.path.isdir(src_dir):
        for fn in os.listdir(src_dir):
            if fn.endswith(".safetensors") or fn == "model.safetensors.index.json":
                continue
            p = os.path.join(src_dir, fn)
            if os.path.isfile(p) and not os.path.exists(os.path.join(directory, fn)):
                shutil.copy(p, os.path.join(directory, fn))
        if extra_config and os.path.exists(os.path.join(directory, "config.json")):
            with open(os.path.join(directory, "config.json")) as f:
                conf = {**json.load(f), **extra_config}
    if not os.path.exists(os.path.join(directory, "config.json")) or extra_config:
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump(conf, f, indent=2)
    open(os.path.join(directory, ".complete"), "w").close()
