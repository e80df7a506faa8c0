"""Small shared helpers: dotted-path plug-in loading, singletons, env report."""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from typing import Any, Callable

_FUNCTION_REGISTRY: dict[str, Callable] = {}


def register_function(name: str, fn: Callable | None = None):
    """Register a callable under a name usable wherever a `--*-path` flag expects a dotted path."""
    if fn is None:
        def deco(f):
            _FUNCTION_REGISTRY[name] = f
            return f
        return deco
    _FUNCTION_REGISTRY[name] = fn
    return fn


def load_function(path: str | Callable | None) -> Callable | None:
    """Resolve `pkg.module.attr`, `pkg.module:attr` or `/file.py:attr`
    (reference: miles/utils/function_registry.py:35)."""
    if path is None or callable(path):
        return path
    if path in _FUNCTION_REGISTRY:
        return _FUNCTION_REGISTRY[path]
    if ":" in path:
        mod_name, attr = path.rsplit(":", 1)
    else:
        mod_name, attr = path.rsplit(".", 1)
    if mod_name.endswith(".py") or os.path.sep in mod_name:
        spec = importlib.util.spec_from_file_location(f"_miles_user_{abs(hash(mod_name))}", mod_name)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
    else:
        mod = importlib.import_module(mod_name)
    obj: Any = mod
    for part in attr.split("."):
        obj = getattr(obj, part)
    return obj


class SingletonMeta(type):
    _instances: dict = {}

    def __call__(cls, *a, **kw):
        if cls not in cls._instances:
            cls._instances[cls] = super().__call__(*a, **kw)
        return cls._instances[cls]

    @classmethod
    def clear(mcs, cls=None):
        if cls is None:
            mcs._instances.clear()
        else:
            mcs._instances.pop(cls, None)


def env_report() -> dict:
    import platform

    import torch

    rep = {
        "python": platform.python_version(),
        "torch": torch.__version__,
        "cuda": torch.version.cuda,
        "cuda_available": torch.cuda.is_available(),
    }
    if torch.cuda.is_available():
        rep["gpu"] = torch.cuda.get_device_name(0)
        rep["gpu_count"] = torch.cuda.device_count()
    for k in ("NCCL_NVLS_ENABLE", "NCCL_DEBUG", "CUDA_VISIBLE_DEVICES", "WORLD_SIZE", "RANK"):
        if k in os.environ:
            rep[k] = os.environ[k]
    return rep


def chunked(seq, n):
    for i in range(0, len(seq), n):
        yield seq[i:i + n]
