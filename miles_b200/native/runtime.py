"""ctypes front-end of the native runtime library (`csrc/runtime.cpp`): KV block allocator, CUDA-VMM arena with
tagged pause/resume, and the router's worker-selection core.  `build()` compiles it with g++ into
`miles_b200/native/_build/libmiles_rt.so`; everything degrades to the pure-python equivalents when the library
has not been built (CPU-only checkouts)."""
from __future__ import annotations

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "runtime.cpp")
SOURCES = [SRC, os.path.join(HERE, "csrc", "codec.cpp")]
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(BUILD_DIR, "libmiles_rt.so")

_lib = None


def build(force: bool = False) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < max(os.path.getmtime(f) for f in SOURCES):
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        subprocess.check_call([cxx, "-O2", "-std=c++17", "-shared", "-fPIC", *SOURCES, "-o", LIB_PATH, "-ldl", "-lpthread"])
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not built; run miles_b200.native.runtime.build()")
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, u64, i64, cp = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint64, ctypes.c_int64, ctypes.c_char_p
        ip = ctypes.POINTER(ctypes.c_int32)
        sigs = {
            "mbrt_alloc_create": (vp, [i32]), "mbrt_alloc_destroy": (None, [vp]), "mbrt_alloc_num_free": (i32, [vp]),
            "mbrt_alloc_take": (i32, [vp, i32, ip]), "mbrt_alloc_share": (None, [vp, ip, i32]),
            "mbrt_alloc_release": (i32, [vp, ip, i32]), "mbrt_alloc_reset": (None, [vp]),
            "mbrt_driver_available": (i32, []), "mbrt_arena_create": (vp, [i32]), "mbrt_arena_malloc": (u64, [vp, u64, cp]),
            "mbrt_arena_free": (i32, [vp, u64]), "mbrt_arena_pause": (i64, [vp, cp, i32]), "mbrt_arena_resume": (i64, [vp, cp]),
            "mbrt_arena_mapped_bytes": (u64, [vp]), "mbrt_arena_destroy": (None, [vp]),
            "mbrt_router_create": (vp, [i32]), "mbrt_router_destroy": (None, [vp]), "mbrt_router_add_worker": (i32, [vp]),
            "mbrt_router_set_health": (None, [vp, i32, i32]), "mbrt_router_pick": (i32, [vp, i32, cp]),
            "mbrt_router_done": (None, [vp, i32]), "mbrt_router_active": (i32, [vp, i32]),
            "mbrt_xxh64": (u64, [vp, u64, u64]), "mbrt_delta_bound": (u64, [u64]),
            "mbrt_delta_encode": (i64, [vp, vp, u64, i32, vp, u64]), "mbrt_delta_decode": (i64, [vp, u64, vp, vp, u64]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except Exception:
        return False


def _arr(blocks):
    return (ctypes.c_int32 * len(blocks))(*blocks)


class NativeBlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._h = lib().mbrt_alloc_create(num_blocks)

    @property
    def num_free(self) -> int:
        return lib().mbrt_alloc_num_free(self._h)

    def alloc(self, n: int):
        out = (ctypes.c_int32 * max(n, 1))()
        if lib().mbrt_alloc_take(self._h, n, out) != 0:
            return None
        return list(out[:n])

    def share(self, blocks):
        lib().mbrt_alloc_share(self._h, _arr(blocks), len(blocks))

    def release(self, blocks):
        if blocks and lib().mbrt_alloc_release(self._h, _arr(blocks), len(blocks)) < 0:
            raise AssertionError("double release of a KV block")

    def reset(self):
        lib().mbrt_alloc_reset(self._h)

    def __del__(self):
        try:
            lib().mbrt_alloc_destroy(self._h)
        except Exception:
            pass


class VmmArena:
    """Tagged GPU allocations whose physical pages can be released and restored at stable addresses."""

    def __init__(self, device: int = 0):
        if not lib().mbrt_driver_available():
            raise RuntimeError("CUDA driver not available")
        import torch

        torch.cuda.init()
        torch.zeros(1, device=f"cuda:{device}")  # make sure the primary context exists and is current
        self.device = device
        self._h = lib().mbrt_arena_create(device)
        if not self._h:
            raise RuntimeError("failed to create the VMM arena")
        self._keep = {}

    def empty(self, shape, dtype, tag: str = "default"):
        """A torch tensor backed by arena memory (through the CUDA array interface)."""
        import numpy as np
        import torch

        numel = int(np.prod(shape)) if len(shape) else 1
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(numel * esize, 1)
        ptr = lib().mbrt_arena_malloc(self._h, nbytes, tag.encode())
        if not ptr:
            raise MemoryError(f"arena allocation of {nbytes} bytes failed")

        class _Holder:
            pass

        h = _Holder()
        h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
        t = torch.as_tensor(h, device=f"cuda:{self.device}").view(dtype)[:numel].view(*shape)
        self._keep[int(ptr)] = h
        t._arena_ptr = int(ptr)
        return t

    def free(self, tensor):
        ptr = getattr(tensor, "_arena_ptr", None)
        if ptr is not None:
            lib().mbrt_arena_free(self._h, ptr)
            self._keep.pop(ptr, None)

    def pause(self, tag: str = "", keep_contents: bool = False) -> int:
        n = lib().mbrt_arena_pause(self._h, tag.encode(), int(keep_contents))
        if n < 0:
            raise RuntimeError("arena pause failed")
        return n

    def resume(self, tag: str = "") -> int:
        n = lib().mbrt_arena_resume(self._h, tag.encode())
        if n < 0:
            raise RuntimeError(f"arena resume failed ({n})")
        return n

    @property
    def mapped_bytes(self) -> int:
        return lib().mbrt_arena_mapped_bytes(self._h)

    def close(self):
        if self._h:
            lib().mbrt_arena_destroy(self._h)
            self._h = None


POLICIES = {"least_active": 0, "round_robin": 1, "consistent_hashing": 2, "random": 3}


class NativeRouterCore:
    def __init__(self, workers: int = 0):
        self._h = lib().mbrt_router_create(workers)

    def add_worker(self) -> int:
        return lib().mbrt_router_add_worker(self._h)

    def set_health(self, w: int, ok: bool):
        lib().mbrt_router_set_health(self._h, w, int(ok))

    def pick(self, policy: str = "least_active", key: str | None = None) -> int:
        return lib().mbrt_router_pick(self._h, POLICIES[policy], (key or "").encode())

    def done(self, w: int):
        lib().mbrt_router_done(self._h, w)

    def active(self, w: int) -> int:
        return lib().mbrt_router_active(self._h, w)

    def __del__(self):
        try:
            lib().mbrt_router_destroy(self._h)
        except Exception:
            pass


# ---- byte codecs (csrc/codec.cpp) ---------------------------------------------------------------------------------

def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data) if a is not None else None


def xxh64(data, seed: int = 0) -> int:
    """XXH64 of a bytes-like object or a numpy array's bytes."""
    import numpy as np

    a = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return int(lib().mbrt_xxh64(_ptr(a) if a.size else None, a.size, seed))


def delta_encode(cur, base=None, elem: int = 2) -> bytes:
    """`cur` (XOR `base` when given) → byte planes → zero-run-length.  Arrays of equal byte length, a multiple of `elem`."""
    import numpy as np

    c = np.ascontiguousarray(cur).view(np.uint8).reshape(-1)
    b = np.ascontiguousarray(base).view(np.uint8).reshape(-1) if base is not None else None
    assert b is None or b.size == c.size, "base and current tensors differ in size"
    out = np.empty(int(lib().mbrt_delta_bound(c.size)), dtype=np.uint8)
    n = lib().mbrt_delta_encode(_ptr(c), _ptr(b), c.size, elem, _ptr(out), out.size)
    if n < 0:
        raise ValueError("delta_encode: inconsistent arguments")
    return out[:n].tobytes()


def delta_decode(blob: bytes, nbytes: int, base=None):
    """Inverse of `delta_encode` → uint8 numpy array of `nbytes`."""
    import numpy as np

    e = np.frombuffer(blob, dtype=np.uint8)
    b = np.ascontiguousarray(base).view(np.uint8).reshape(-1) if base is not None else None
    assert b is None or b.size == nbytes
    out = np.empty(nbytes, dtype=np.uint8)
    if lib().mbrt_delta_decode(_ptr(e), e.size, _ptr(b), _ptr(out), nbytes) != nbytes:
        raise ValueError("delta_decode: malformed stream")
    return out
