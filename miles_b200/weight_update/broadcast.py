"""Disaggregated weight sync: broadcast HF-named buckets from trainer rank 0 to engine processes.

Reference protocol (weight_update/protocols/broadcast.py:21-208): an ad-hoc process group {trainer source rank} ∪
{every engine GPU}; for each bucket the engines are first told names/dtypes/shapes over HTTP
(`update_weights_from_distributed`), then the tensors arrive with `dist.broadcast(src=0)` — one call per tensor, or one
byte-flattened bucket in `broadcast_packed` mode.  Here the group is built directly on a `TCPStore`
(`make_group`), so it is independent of each side's default process group; over NVSwitch the NCCL broadcast runs at
link rate, and the packed mode turns a bucket into a single collective (launch latency, not bandwidth, is what
per-tensor broadcasts of small tensors pay for).
"""
from __future__ import annotations

import datetime
import threading
from typing import Any

import torch
import torch.distributed as dist

from .hf_iterator import iter_hf_weights

_GROUPS: dict[str, Any] = {}
ALIGN = 256     # byte alignment of each tensor inside a packed bucket


def make_group(backend: str, host: str, port: int, rank: int, world: int, timeout_s: float = 300.0, name: str = "weight_sync"):
    """A process group of its own (not a sub-group of the default one), rendezvous over a TCPStore at host:port."""
    store = dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s),
                          wait_for_workers=False)
    store = dist.PrefixStore(name, store)
    to = datetime.timedelta(seconds=timeout_s)
    if backend == "nccl":
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = to
        pg = dist.ProcessGroupNCCL(store, rank, world, opts)
    else:
        pg = dist.ProcessGroupGloo(store, rank, world, to)
    _GROUPS[name] = pg
    return pg


def get_group(name: str = "weight_sync"):
    return _GROUPS.get(name)


def destroy_group(name: str = "weight_sync"):
    _GROUPS.pop(name, None)


def _bcast(pg, t: torch.Tensor, src: int = 0):
    opts = dist.BroadcastOptions()
    opts.rootRank = src
    opts.rootTensor = 0
    pg.broadcast([t], opts).wait()


def bucket_meta(bucket: list[tuple[str, torch.Tensor]]) -> dict:
    return {"names": [n for n, _ in bucket], "dtypes": [str(t.dtype).replace("torch.", "") for _, t in bucket],
            "shapes": [list(t.shape) for _, t in bucket]}


def packed_layout(meta: dict) -> tuple[list[int], int]:
    """Byte offset of every tensor inside the flattened bucket and the bucket's size."""
    offs, off = [], 0
    for dt, shape in zip(meta["dtypes"], meta["shapes"]):
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty(0, dtype=getattr(torch, dt)).element_size()
        offs.append(off)
        off += (nb + ALIGN - 1) // ALIGN * ALIGN
    return offs, off


def send_bucket(pg, bucket: list[tuple[str, torch.Tensor]], packed: bool, device) -> int:
    n = 0
    if packed:
        meta = bucket_meta(bucket)
        offs, size = packed_layout(meta)
        flat = torch.empty(size, dtype=torch.uint8, device=device)
        for (name, t), o in zip(bucket, offs):
            b = t.contiguous().view(-1).view(torch.uint8)
            flat[o:o + b.numel()].copy_(b)
            n += b.numel()
        _bcast(pg, flat)
    else:
        for _, t in bucket:
            t = t.contiguous().to(device)
            _bcast(pg, t)
            n += t.numel() * t.element_size()
    return n


def recv_bucket(pg, meta: dict, packed: bool, device) -> list[tuple[str, torch.Tensor]]:
    out = []
    if packed:
        offs, size = packed_layout(meta)
        flat = torch.empty(size, dtype=torch.uint8, device=device)
        _bcast(pg, flat)
        for name, dt, shape, o in zip(meta["names"], meta["dtypes"], meta["shapes"], offs):
            dtype = getattr(torch, dt)
            numel = 1
            for s in shape:
                numel *= s
            nb = numel * torch.empty(0, dtype=dtype).element_size()
            out.append((name, flat[o:o + nb].view(dtype).view(shape)))
    else:
        for name, dt, shape in zip(meta["names"], meta["dtypes"], meta["shapes"]):
            t = torch.empty(shape, dtype=getattr(torch, dt), device=device)
            _bcast(pg, t)
            out.append((name, t))
    return out


class RemoteEngine:
    """Handle of an engine server reached over HTTP (the endpoints of `miles_b200.engine.server`)."""

    def __init__(self, url: str, timeout: float = 600.0):
        self.url, self.timeout = url.rstrip("/"), timeout

    def post(self, endpoint: str, body: dict | None = None) -> dict:
        import requests

        r = requests.post(f"{self.url}/{endpoint.lstrip('/')}", json=body or {}, timeout=self.timeout)
        r.raise_for_status()
        return r.json() if r.content else {}

    def get(self, endpoint: str) -> dict:
        import requests

        r = requests.get(f"{self.url}/{endpoint.lstrip('/')}", timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    # the subset of the engine API the updater's session frame uses
    def pause_generation(self, mode="retract"):
        return self.post("pause_generation", {"mode": mode})

    def continue_generation(self):
        return self.post("continue_generation")

    def flush_cache(self):
        return self.post("flush_cache")

    def update_weight_version(self, v):
        return self.post("update_weight_version", {"weight_version": int(v)})

    def get_weight_version(self):
        return int(self.get("get_weight_version")["weight_version"])

    def init_weights_update_group(self, **kw):
        return self.post("init_weights_update_group", kw)

    def update_weights_from_distributed(self, **kw):
        return self.post("update_weights_from_distributed", kw)

    def update_weights_from_disk(self, path, weight_version=None):
        return self.post("update_weights_from_disk", {"model_path": path, "weight_version": weight_version})


def connect(updater, host: str = "127.0.0.1", port: int = 29600, backend: str | None = None, group_name: str = "weight_sync"):
    """Build the {trainer rank 0} ∪ {engines} group.  Engine i takes rank 1 + i·gpus_per_engine + its local rank."""
    engines = updater.engines
    per = getattr(updater.args, "rollout_num_gpus_per_engine", 1) or 1
    world = 1 + per * len(engines)
    backend = backend or ("nccl" if updater.actor.device.type == "cuda" else "gloo")
    threads = []
    if updater._is_leader():
        for i, e in enumerate(engines):
            kw = dict(master_address=host, master_port=port, rank_offset=1 + i * per, world_size=world, group_name=group_name,
                      backend=backend)
            t = threading.Thread(target=e.init_weights_update_group, kwargs=kw, daemon=True)
            t.start()
            threads.append(t)
        pg = make_group(backend, host, port, 0, world, name=group_name)
        for t in threads:
            t.join()
        updater.connected_engines_hash = hash(tuple(getattr(e, "url", id(e)) for e in engines))
        return pg
    return None


def broadcast_buckets(updater, group_name: str = "weight_sync") -> int:
    """Stream every bucket: all trainer ranks take part in the shard gathers, rank 0 alone talks to the engines."""
    args = updater.args
    packed = getattr(updater, "packed", False) or getattr(args, "broadcast_packed", False)
    leader = updater._is_leader()
    pg = get_group(group_name)
    if leader and pg is None:
        pg = connect(updater, getattr(args, "update_weight_master_addr", "127.0.0.1"),
                     getattr(args, "update_weight_master_port", 29600), group_name=group_name)
    n = 0
    size = getattr(args, "update_weight_buffer_size", 512 << 20)
    for bucket in iter_hf_weights(updater.actor, bucket_bytes=size, quant=updater.quant):
        if not leader:
            continue
        meta = bucket_meta(bucket)
        threads = []
        for e in updater.engines:
            kw = dict(meta, group_name=group_name, load_format="flattened_bucket" if packed else None)
            t = threading.Thread(target=e.update_weights_from_distributed, kwargs=kw, daemon=True)
            t.start()
            threads.append(t)
        n += send_bucket(pg, bucket, packed, updater.actor.device)
        for t in threads:
            t.join()
    return n
