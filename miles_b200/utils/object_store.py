"""put / get / remove of rollout batches between the rollout executor and trainer ranks.

In-process dict by default; a directory-backed store (one pickle per key, atomic rename) lets
separate processes on one box exchange batches.  The reference's store sits on Ray's object store or
Mooncake (miles/utils/object_store.py:112-245); neither is needed on a single NVSwitch box.
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


def configure(directory: str | None):
    global _DIR
    _DIR = directory
    if directory:
        os.makedirs(directory, exist_ok=True)


def put(obj: Any, key: str | None = None) -> str:
    key = key or uuid.uuid4().hex
    if _DIR:
        tmp = os.path.join(_DIR, f".{key}.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(obj, f, protocol=pickle.HIGHEST_PROTOCOL)
        os.replace(tmp, os.path.join(_DIR, key))
    else:
        with _LOCK:
            _LOCAL[key] = obj
    return key


def get(key: str) -> Any:
    if _DIR and os.path.exists(os.path.join(_DIR, key)):
        with open(os.path.join(_DIR, key), "rb") as f:
            return pickle.load(f)
    with _LOCK:
        return _LOCAL[key]


def remove(key: str) -> None:
    if _DIR:
        try:
            os.remove(os.path.join(_DIR, key))
        except FileNotFoundError:
            pass
    with _LOCK:
        _LOCAL.pop(key, None)
