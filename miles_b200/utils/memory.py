"""Moving tensors out of and back into GPU memory for colocated train/rollout hand-off.

Two mechanisms:
* `offload_tensors` / `onload_tensors`: keep the python tensor objects, swap their storage for a
  pinned host copy (the torch-native `offload.py` of the reference,
  miles/backends/training_utils/torch_native/offload.py:1-29).
* `miles_b200.native.runtime.VmmArena`: a C++ CUDA-VMM arena with tagged pause/resume that frees
  the physical pages but keeps virtual addresses stable (the role `torch_memory_saver` plays for the
  reference), so CUDA graphs and peer mappings survive a sleep/wake cycle.  `make_arena` gives the trainer one when
  `--offload-train` is on and the native runtime is built; optimizer state then lives in it under the tag "optimizer".
"""
from __future__ import annotations

import torch


def offload_tensors(tensors: list[torch.Tensor]) -> list[tuple[torch.Tensor, torch.Tensor]]:
    saved = []
    for t in tensors:
        if not t.is_cuda:
            saved.append((t, None))
            continue
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t, non_blocking=True)
        saved.append((t, host))
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for t, host in saved:
        if host is not None:
            t._offload_device = t.device
            t.data = torch.empty(0, dtype=t.dtype, device=t.device)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return saved


def onload_tensors(saved: list[tuple[torch.Tensor, torch.Tensor]]):
    for t, host in saved:
        if host is None:
            continue
        t.data = host.to(t._offload_device, non_blocking=True)
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def make_arena(device) -> "object | None":
    """A VMM arena on `device`, or None where it cannot exist (CPU, native runtime not built, driver without VMM)."""
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        return None
    try:
        from ..native import runtime as rt

        if not rt.available():
            return None
        return rt.VmmArena(dev.index if dev.index is not None else torch.cuda.current_device())
    except Exception:
        return None


def gpu_memory_report(device=None) -> dict:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info(device)
    return {
        "free_gb": free / 2**30,
        "total_gb": total / 2**30,
        "allocated_gb": torch.cuda.memory_allocated(device) / 2**30,
        "reserved_gb": torch.cuda.memory_reserved(device) / 2**30,
    }
