"""put / get / remove of rollout batches between the rollout executor and trainer ranks.

Three backends behind the same calls: an in-process dict (default); a directory (one file per key, atomic rename) for
separate processes on one box; a key-value store object with `set(key, bytes)` / `get(key)` (a `torch.distributed.TCPStore`
reaches other nodes) chosen with `configure(store=…)`.  Values that are training batches (dicts of per-sample lists) are
written with the typed ragged codec (`utils/ragged_codec.py`: flat arrays + offsets for the per-token fields), everything
else with pickle.  The reference's store sits on Ray's object store or Mooncake with typed-ragged encodings
(miles/utils/object_store.py:112-245).
"""
from __future__ import annotations

import os
import pickle
import threading
import uuid
from typing import Any

_LOCAL: dict[str, Any] = {}
_LOCK = threading.Lock()
_DIR: str | None = os.environ.get("MILES_OBJECT_STORE_DIR")
_STORE = None                     # an object with set(key, bytes) / get(key) -> bytes / delete_key(key)
_BATCH_KEYS = ("tokens", "loss_masks", "rollout_log_probs")


def configure(directory: str | None = None, store=None):
    global _DIR, _STORE
    _DIR, _STORE = directory, store
    if directory:
        os.makedirs(directory, exist_ok=True)


def _dumps(obj: Any) -> bytes:
    """Training batches ({"tokens": [[…], …], "loss_masks": …, …}) as typed ragged arrays; anything else pickled."""
    if isinstance(obj, dict) and "tokens" in obj and isinstance(obj["tokens"], list):
        import numpy as np

        enc = {"__ragged_batch__": True, "rest": {}}
        for k, v in obj.items():
            if isinstance(v, list) and v and all(isinstance(x, list) for x in v) and all(not x or isinstance(x[0], (int, float)) for x in v):
                is_int = all(isinstance(y, int) for x in v for y in x[:1])
                enc[k] = (np.fromiter((len(x) for x in v), dtype=np.int64, count=len(v)),
                          np.concatenate([np.asarray(x, dtype=np.int64 if is_int else np.float32) for x in v]) if any(v) else
                          np.zeros(0, dtype=np.int64 if is_int else np.float32))
            else:
                enc["rest"][k] = v
        return b"B" + pickle.dumps(enc, protocol=5)
    return b"P" + pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)


def _loads(blob: bytes) -> Any:
    if blob[:1] == b"P":
        return pickle.loads(blob[1:])
    enc = pickle.loads(blob[1:])
    out = dict(enc["rest"])
    for k, v in enc.items():
        if k in ("__ragged_batch__", "rest"):
            continue
        lens, data = v
        at, rows = 0, []
        for n in lens.tolist():
            rows.append(data[at:at + n].tolist())
            at += n
        out[k] = rows
    return out


def put(obj: Any, key: str | None = None) -> str:
    key = key or uuid.uuid4().hex
    if _STORE is not None:
        _STORE.set(f"objstore/{key}", _dumps(obj))
    elif _DIR:
        tmp = os.path.join(_DIR, f".{key}.tmp")
        with open(tmp, "wb") as f:
            f.write(_dumps(obj))
        os.replace(tmp, os.path.join(_DIR, key))
    else:
        with _LOCK:
            _LOCAL[key] = obj
    return key


def get(key: str) -> Any:
    if _STORE is not None:
        return _loads(bytes(_STORE.get(f"objstore/{key}")))
    if _DIR and os.path.exists(os.path.join(_DIR, key)):
        with open(os.path.join(_DIR, key), "rb") as f:
            return _loads(f.read())
    with _LOCK:
        return _LOCAL[key]


def remove(key: str) -> None:
    if _STORE is not None:
        try:
            _STORE.delete_key(f"objstore/{key}")
        except Exception:
            pass
        return
    if _DIR:
        try:
            os.remove(os.path.join(_DIR, key))
        except FileNotFoundError:
            pass
    with _LOCK:
        _LOCAL.pop(key, None)
