"""Typed ragged codec for batches of samples: the large per-token fields travel as flat arrays with offsets, not as
Python lists.

A rollout batch is a few hundred samples whose bulk is per-token data — token ids, loss masks, sampling log-probs, teacher
log-probs, routed experts.  Pickling them as lists of Python numbers costs an object per token (seconds per batch when
every rank gathers every sample); the reference ships such fields through typed, ragged encodings of its object store
(miles/utils/object_store.py:112-245).  Here every known ragged field of all samples is concatenated into ONE typed numpy
array plus an offsets array (`None` and "empty" are kept apart), n-d arrays are stored with their shapes, and only the
small remainder of each sample goes through pickle.  Arrays pickle by buffer (protocol 5), so encode → gather → decode
moves bytes, not objects.
"""
from __future__ import annotations

import pickle
import zlib
from typing import Any

import numpy as np

# field → dtype of the flat array
RAGGED_FIELDS = {"tokens": np.int32, "loss_mask": np.uint8, "rollout_log_probs": np.float32, "teacher_log_probs": np.float32,
                 "opd_reverse_kl": np.float32, "witness_ids": np.int64}
ND_FIELDS = ("rollout_routed_experts",)
MAGIC = b"MRC1"


def encode_dicts(rows: list[dict]) -> dict[str, Any]:
    """`rows`: sample dicts (e.g. `Sample.to_dict()` with arrays left as arrays, or any dicts with these field names)."""
    out: dict[str, Any] = {"n": len(rows)}
    rest = []
    for name, dt in RAGGED_FIELDS.items():
        lens = np.full(len(rows), -1, dtype=np.int64)              # −1: the field is None / absent
        parts = []
        for i, r in enumerate(rows):
            v = r.get(name)
            if v is not None:
                a = np.asarray(v, dtype=dt)
                lens[i] = a.size
                parts.append(a.reshape(-1))
        if (lens >= 0).any():
            out[f"r.{name}.len"] = lens
            out[f"r.{name}.data"] = np.concatenate(parts) if parts else np.zeros(0, dtype=dt)
    for name in ND_FIELDS:
        shapes, parts, dtype = [], [], None
        for r in rows:
            v = r.get(name)
            if isinstance(v, dict) and "__nd__" in v:                   # the base64 form of `Sample.to_dict`
                import base64

                v = np.frombuffer(base64.b64decode(v["__nd__"]), dtype=v["dtype"]).reshape(v["shape"])
            if v is None:
                shapes.append(None)
            else:
                a = np.ascontiguousarray(v)
                dtype = dtype or a.dtype
                shapes.append(a.shape)
                parts.append(a.reshape(-1).astype(dtype, copy=False))
        if parts:
            out[f"n.{name}.shapes"] = shapes
            out[f"n.{name}.data"] = np.concatenate(parts)
    skip = set(RAGGED_FIELDS) | set(ND_FIELDS)
    for r in rows:
        rest.append({k: v for k, v in r.items() if k not in skip})
    out["rest"] = rest
    return out


def decode_dicts(enc: dict[str, Any]) -> list[dict]:
    n = enc["n"]
    rows = [dict(r) for r in enc["rest"]]
    for name, dt in RAGGED_FIELDS.items():
        lens = enc.get(f"r.{name}.len")
        if lens is None:
            for r in rows:
                r.setdefault(name, None)
            continue
        data = enc[f"r.{name}.data"]
        at = 0
        for i in range(n):
            L = int(lens[i])
            if L < 0:
                rows[i][name] = None
            else:
                rows[i][name] = data[at:at + L].tolist()
                at += L
    for name in ND_FIELDS:
        shapes = enc.get(f"n.{name}.shapes")
        if shapes is None:
            for r in rows:
                r.setdefault(name, None)
            continue
        data = enc[f"n.{name}.data"]
        at = 0
        for i, shp in enumerate(shapes):
            if shp is None:
                rows[i][name] = None
            else:
                size = int(np.prod(shp)) if len(shp) else 1
                rows[i][name] = data[at:at + size].reshape(shp).copy()
                at += size
    return rows


def dumps(rows: list[dict], compress: bool = False) -> bytes:
    body = pickle.dumps(encode_dicts(rows), protocol=5)
    return MAGIC + (b"Z" + zlib.compress(body, 1) if compress else b"R" + body)


def loads(blob: bytes) -> list[dict]:
    assert blob[:4] == MAGIC, "not a ragged-codec blob"
    body = blob[5:]
    return decode_dicts(pickle.loads(zlib.decompress(body) if blob[4:5] == b"Z" else body))


def encode_groups(groups: list[list]) -> dict[str, Any]:
    """Groups of `Sample` objects → one encoding (group sizes kept)."""
    rows = []
    for g in groups:
        for s in g:
            d = s.to_dict() if hasattr(s, "to_dict") else dict(s)
            v = getattr(s, "rollout_routed_experts", None)
            if v is not None:
                d["rollout_routed_experts"] = v                      # keep the array: no base64 detour
            rows.append(d)
    enc = encode_dicts(rows)
    enc["group_sizes"] = [len(g) for g in groups]
    return enc


def decode_groups(enc: dict[str, Any], sample_cls) -> list[list]:
    rows = decode_dicts(enc)
    out, at = [], 0
    for n in enc["group_sizes"]:
        out.append([sample_cls.from_dict(r) for r in rows[at:at + n]])
        at += n
    return out
