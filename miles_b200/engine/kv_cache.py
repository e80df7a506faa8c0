"""Paged KV cache: fixed-size blocks, per-request block tables, a free-list allocator.

The allocator has a C++ implementation (`miles_b200.native`, lock-free free list + ref counts for
shared prefixes) that is used when the native runtime library is built; the python class below is
the same algorithm and the CPU-test path.  The engine the reference drives (SGLang, radix/paged KV)
is external to it; sizing follows its `--sglang-mem-fraction-static` knob.
"""
from __future__ import annotations

import torch


class BlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self.free: list[int] = list(range(num_blocks - 1, -1, -1))
        self.refcnt = [0] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self.free)

    def alloc(self, n: int) -> list[int] | None:
        if n > len(self.free):
            return None
        out = [self.free.pop() for _ in range(n)]
        for b in out:
            self.refcnt[b] = 1
        return out

    def share(self, blocks: list[int]):
        for b in blocks:
            self.refcnt[b] += 1

    def release(self, blocks: list[int]):
        for b in blocks:
            self.refcnt[b] -= 1
            if self.refcnt[b] == 0:
                self.free.append(b)
            assert self.refcnt[b] >= 0

    def reset(self):
        self.free = list(range(self.num_blocks - 1, -1, -1))
        self.refcnt = [0] * self.num_blocks


def make_allocator(num_blocks: int):
    try:
        from ..native import runtime as rt

        if rt.available():
            return rt.NativeBlockAllocator(num_blocks)
    except Exception:
        pass
    return BlockAllocator(num_blocks)


class KVCache:
    """Per-layer K and V tensors of shape [num_blocks, block_size, Hkv, D]."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, num_kv_heads: int, head_dim: int,
                 dtype, device, layer_ids: list[int] | None = None):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.shape = (num_blocks, block_size, num_kv_heads, head_dim)
        self.dtype, self.device = dtype, device
        self.layer_ids = layer_ids if layer_ids is not None else list(range(num_layers))
        self.layers: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.allocate()

    def allocate(self):
        for l in self.layer_ids:
            self.layers[l] = (torch.zeros(self.shape, dtype=self.dtype, device=self.device),
                              torch.zeros(self.shape, dtype=self.dtype, device=self.device))

    def free(self):
        """Release the cache memory (engine `release_memory_occupation(tags=['kv_cache'])`)."""
        self.layers = {}
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    @property
    def allocated(self) -> bool:
        return bool(self.layers)

    def bytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return 2 * n * len(self.layer_ids) * torch.empty((), dtype=self.dtype).element_size()

    @staticmethod
    def blocks_for_budget(bytes_budget: int, num_layers: int, block_size: int, num_kv_heads: int, head_dim: int, dtype) -> int:
        per = 2 * num_layers * block_size * num_kv_heads * head_dim * torch.empty((), dtype=dtype).element_size()
        return max(1, bytes_budget // per)
