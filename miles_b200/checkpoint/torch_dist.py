"""Megatron `torch_dist` checkpoints (torch.distributed.checkpoint directories).

The reference's Megatron backend saves and loads `iter_XXXXXXX/` directories in `torch_dist` format
(`dist_checkpointing`, used through `--load/--save/--ref-load`; converters `tools/convert_hf_to_torch_dist.py`,
`tools/convert_torch_dist_to_hf.py`).  A `torch_dist` directory is a DCP store: `.metadata` plus `__*_*.distcp`
shard files, holding Megatron-named full tensors (`decoder.layers.0.self_attention.linear_qkv.weight`, …).
This module reads such a directory into a flat `{megatron_name: tensor}` dict without a process group and writes one
from a dict, so that checkpoints move between this package, HF and Megatron without the Megatron runtime.
"""
from __future__ import annotations

import os

import torch


def is_torch_dist_dir(d: str) -> bool:
    return os.path.isdir(d) and os.path.exists(os.path.join(d, ".metadata"))


def has_per_layer_names(d: str) -> bool:
    """True when the store names decoder layers one by one (`decoder.layers.<i>.…`); Megatron-core may instead stack all
    layers of a block under one entry with a leading layer axis, which `load_state` unstacks."""
    import re

    import torch.distributed.checkpoint as dcp

    keys = dcp.FileSystemReader(d).read_metadata().state_dict_metadata.keys()
    layered = [k for k in keys if ".layers." in k and "optimizer" not in k]
    return all(re.search(r"\.layers\.\d+\.", k) for k in layered)


def find_iteration_dir(root: str) -> str:
    """`root` may be the iteration directory itself or a Megatron checkpoint root with
    `latest_checkpointed_iteration.txt`."""
    if is_torch_dist_dir(root):
        return root
    tracker = os.path.join(root, "latest_checkpointed_iteration.txt")
    if os.path.exists(tracker):
        it = open(tracker).read().strip()
        d = os.path.join(root, "release" if it == "release" else f"iter_{int(it):07d}")
        if is_torch_dist_dir(d):
            return d
    raise FileNotFoundError(f"no torch_dist checkpoint under {root}")


def load_state(d: str, prefix_filter: tuple[str, ...] = ("optimizer", "rng", "_extra_state")) -> dict[str, torch.Tensor]:
    """Read every tensor entry of the DCP directory (skipping optimizer / rng / TE extra state)."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    d = find_iteration_dir(d)
    reader = dcp.FileSystemReader(d)
    meta = reader.read_metadata()
    sd = {}
    for name, m in meta.state_dict_metadata.items():
        if not isinstance(m, TensorStorageMetadata):
            continue
        if any(p in name for p in prefix_filter):
            continue
        sd[name] = torch.empty(m.size, dtype=m.properties.dtype)
    dcp.load(sd, storage_reader=reader, no_dist=True)
    import re

    out = {}
    for k, v in sd.items():
        k = k[len("model."):] if k.startswith("model.") else k      # Megatron nests weights under "model."
        k = k[len("module.module."):] if k.startswith("module.module.") else k
        # Megatron-core may store all layers of a block as ONE entry with a leading layer axis, and grouped experts as
        # one entry with a leading expert axis: split both into the per-layer / per-expert names
        layered = [(k, v)]
        if ".layers." in k and not re.search(r"\.layers\.\d+\.", k):
            layered = [(k.replace(".layers.", f".layers.{i}."), v[i]) for i in range(v.shape[0])]
        for k2, v2 in layered:
            if ".experts.experts." in k2 and not re.search(r"\.weight\d+$", k2):
                for e in range(v2.shape[0]):
                    out[k2.replace(".experts.experts.", ".experts.") + str(e)] = v2[e]
            else:
                out[k2] = v2
    return out


def save_state(state: dict[str, torch.Tensor], d: str, iteration: int | None = None) -> str:
    """Write `{megatron_name: full tensor}` as a single-writer DCP directory (plus Megatron's tracker file when an
    iteration number is given)."""
    import torch.distributed.checkpoint as dcp

    if iteration is not None:
        root = d
        d = os.path.join(root, f"iter_{iteration:07d}")
    os.makedirs(d, exist_ok=True)
    sd = {f"model.{k}": v.detach().cpu().contiguous() for k, v in state.items()}
    dcp.save(sd, storage_writer=dcp.FileSystemWriter(d, single_file_per_rank=True, thread_count=1), no_dist=True)
    if iteration is not None:
        with open(os.path.join(root, "latest_checkpointed_iteration.txt"), "w") as f:
            f.write(str(iteration))
    return d
