"""Disk-delta weight transfer and HF snapshot publishing.

Reference: weight_update/protocols/delta.py:69-470 (engines that cannot join a process group — other clusters,
serving fleets — follow training by applying per-version *deltas* from shared storage; codec with zstd + checksums in
miles/utils/disk_delta.py) and weight_update/snapshot_publisher.py:26-99 (periodic full HF safetensors export with an
atomically updated `latest` pointer).

Delta format (one directory per version `v{N}`):
    manifest.json   {"version", "base_version", "tensors": {name: {"dtype", "shape", "kind", "file", "nbytes", "crc32"}}}
    <file>.bin      payload: `kind == "full"`  raw tensor bytes
                             `kind == "xor"`   bytes of (new XOR base) — bf16 weights move little per step, so the XOR
                                               is mostly zero bytes and compresses well
    Payloads are compressed when that helps; "codec" records how: "zrle" (the native runtime's byte-plane + zero-run-length
    coder, `native/csrc/codec.cpp`: one pass at hundreds of MB/s, made for XOR deltas), "zrle+zlib" (the same, then zlib: the
    smallest), "zlib", or "raw".  Checksums: crc32 always, XXH64 ("xxh64") too when the native runtime is built.
A reader applies deltas in order on top of the version it holds; a checksum mismatch or a missing base is an error the
caller answers by loading the newest full snapshot.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Iterable

import torch

from ..checkpoint import hf_io


def _bytes_of(t: torch.Tensor) -> bytes:
    return t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()


def _native():
    try:
        from ..native import runtime as rt

        return rt if rt.available() else None
    except Exception:
        return None


def _from_bytes(b: bytes, dtype, shape) -> torch.Tensor:
    return torch.frombuffer(bytearray(b), dtype=torch.uint8).view(dtype).view(shape).clone()


class DeltaWriter:
    """Trainer side: keeps the last published tensors (host memory) and writes XOR deltas against them."""

    def __init__(self, root: str, full_every: int = 10, compress: bool = True, codec: str = "auto"):
        """`codec`: "auto" (zrle+zlib with the native runtime, else zlib), "zrle", "zrle+zlib", "zlib" or "raw"."""
        self.root, self.full_every, self.compress = root, full_every, compress
        rt = _native()
        if codec == "auto":
            codec = "zrle+zlib" if rt is not None else "zlib"
        if codec.startswith("zrle") and rt is None:
            raise RuntimeError("the zrle codec needs the native runtime (miles_b200.native.runtime.build())")
        self.codec = codec if compress else "raw"
        self.base: dict[str, torch.Tensor] = {}
        self.base_version: int | None = None
        self.published = 0
        os.makedirs(root, exist_ok=True)

    def publish(self, version: int, named: Iterable[tuple[str, torch.Tensor]]) -> dict:
        d = os.path.join(self.root, f"v{version}")
        tmp = d + ".tmp"
        os.makedirs(tmp, exist_ok=True)
        full = self.base_version is None or (self.full_every and self.published % self.full_every == 0)
        manifest = {"version": version, "base_version": None if full else self.base_version, "tensors": {}}
        raw_bytes = stored = 0
        new_base = {}
        for i, (name, t) in enumerate(named):
            cur = t.detach().contiguous().cpu()
            kind = "full"
            payload = _bytes_of(cur)
            if not full and name in self.base and self.base[name].shape == cur.shape and self.base[name].dtype == cur.dtype:
                x = torch.bitwise_xor(cur.view(torch.uint8), self.base[name].view(torch.uint8))
                payload, kind = x.numpy().tobytes(), "xor"
            raw = _bytes_of(cur)
            crc = zlib.crc32(raw)
            rt = _native()
            codec = "raw"
            if self.codec.startswith("zrle"):
                z = rt.delta_encode(torch.frombuffer(bytearray(payload), dtype=torch.uint8).numpy(), None, max(1, cur.element_size()))
                if self.codec == "zrle+zlib":
                    z2 = zlib.compress(z, 1)
                    if len(z2) < len(payload) and len(z2) < len(z):
                        payload, codec = z2, "zrle+zlib"
                if codec == "raw" and len(z) < len(payload):
                    payload, codec = z, "zrle"
            elif self.codec == "zlib":
                z = zlib.compress(payload, 1)
                if len(z) < len(payload):
                    payload, codec = z, "zlib"
            fn = f"t{i:05d}.bin"
            with open(os.path.join(tmp, fn), "wb") as f:
                f.write(payload)
            manifest["tensors"][name] = {"dtype": str(cur.dtype).replace("torch.", ""), "shape": list(cur.shape), "kind": kind,
                                         "file": fn, "nbytes": len(payload), "crc32": crc, "codec": codec}
            if rt is not None:
                manifest["tensors"][name]["xxh64"] = f"{rt.xxh64(raw):016x}"
            raw_bytes += cur.numel() * cur.element_size()
            stored += len(payload)
            new_base[name] = cur
        with open(os.path.join(tmp, "manifest.json"), "w") as f:
            json.dump(manifest, f)
        os.replace(tmp, d)                      # a version directory appears atomically
        with open(os.path.join(self.root, "latest.tmp"), "w") as f:
            f.write(str(version))
        os.replace(os.path.join(self.root, "latest.tmp"), os.path.join(self.root, "latest"))
        self.base, self.base_version = new_base, version
        self.published += 1
        return {"version": version, "full": bool(full), "raw_bytes": raw_bytes, "stored_bytes": stored}


class DeltaReader:
    """Engine side: holds its current tensors and walks the delta chain up to a target version."""

    def __init__(self, root: str):
        self.root = root
        self.state: dict[str, torch.Tensor] = {}
        self.version: int | None = None

    def latest(self) -> int | None:
        p = os.path.join(self.root, "latest")
        return int(open(p).read().strip()) if os.path.exists(p) else None

    def _manifest(self, version: int) -> dict:
        with open(os.path.join(self.root, f"v{version}", "manifest.json")) as f:
            return json.load(f)

    def _chain(self, target: int) -> list[int]:
        chain, v = [], target
        while True:
            m = self._manifest(v)
            chain.append(v)
            if m["base_version"] is None or m["base_version"] == self.version:
                break
            v = m["base_version"]
        return chain[::-1]

    def update_to(self, target: int | None = None) -> dict[str, torch.Tensor]:
        target = self.latest() if target is None else target
        assert target is not None, "nothing has been published"
        if target == self.version:
            return self.state
        for v in self._chain(target):
            m = self._manifest(v)
            for name, e in m["tensors"].items():
                with open(os.path.join(self.root, f"v{v}", e["file"]), "rb") as f:
                    payload = f.read()
                dtype = getattr(torch, e["dtype"])
                if e["codec"] in ("zlib", "zrle+zlib"):
                    payload = zlib.decompress(payload)
                if e["codec"] in ("zrle", "zrle+zlib"):
                    rt = _native()
                    if rt is None:
                        raise RuntimeError("this delta was written with the zrle codec: build the native runtime to read it")
                    n = 1
                    for d_ in e["shape"]:
                        n *= d_
                    payload = rt.delta_decode(payload, n * torch.empty((), dtype=dtype).element_size()).tobytes()
                if e["kind"] == "xor":
                    assert name in self.state and m["base_version"] == self.version, \
                        f"delta v{v} needs base v{m['base_version']}, reader holds v{self.version}"
                    x = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
                    cur = torch.bitwise_xor(self.state[name].contiguous().view(torch.uint8).view(-1), x).view(dtype).view(e["shape"])
                else:
                    cur = _from_bytes(payload, dtype, e["shape"])
                got = _bytes_of(cur)
                if zlib.crc32(got) != e["crc32"]:
                    raise IOError(f"checksum mismatch for {name} in v{v}")
                rt = _native()
                if rt is not None and "xxh64" in e and f"{rt.xxh64(got):016x}" != e["xxh64"]:
                    raise IOError(f"xxh64 mismatch for {name} in v{v}")
                self.state[name] = cur
            self.version = v
        return self.state


class SnapshotPublisher:
    """Periodic full HF export: `root/step_{N}/` safetensors + config, `root/latest` flipped last; keeps `keep` snapshots."""

    def __init__(self, root: str, cfg, every: int = 1, keep: int = 2, src_dir: str | None = None):
        self.root, self.cfg, self.every, self.keep, self.src_dir = root, cfg, every, keep, src_dir
        os.makedirs(root, exist_ok=True)

    def maybe_publish(self, step: int, bucket_iter, write: bool = True) -> str | None:
        """`bucket_iter`: iterator of HF-named buckets (every trainer rank drives it; only `write` ranks touch disk)."""
        if self.every and step % self.every:
            for _ in bucket_iter:               # collectives inside the iterator still have to run on every rank
                pass
            return None
        d = os.path.join(self.root, f"step_{step}")
        hf_io.save_hf_sharded(d, bucket_iter, self.cfg, write=write, src_dir=self.src_dir)
        if write:
            with open(os.path.join(self.root, "latest.tmp"), "w") as f:
                f.write(f"step_{step}")
            os.replace(os.path.join(self.root, "latest.tmp"), os.path.join(self.root, "latest"))
            snaps = sorted((x for x in os.listdir(self.root) if x.startswith("step_")), key=lambda s: int(s.split("_")[1]))
            for old in snaps[:-self.keep] if self.keep else []:
                import shutil

                shutil.rmtree(os.path.join(self.root, old), ignore_errors=True)
        return d
