"""Adam whose fp32 master weights and moments live in files and stream through the GPU bucket by bucket.

Reference: miles_plugins/optimizers/nvme_stream.py:265-763 (used for models whose optimizer state does not fit beside
the colocated engine: per step ≈ 72 GB read + 144 GB written per GPU in the reference's MiMo run) and the disk offload
of trainer sleep/wake (docs/advanced/disk-offload.md).  State layout: three flat fp32 files per rank
(`master.bin`, `exp_avg.bin`, `exp_avg_sq.bin`) of `numel` floats.  A step walks the flat gradient in buckets:

    read bucket i+1 (background thread, pinned buffer B)   ║   H2D bucket i → AdamW kernel → D2H bucket i (stream)   ║   write bucket i−1

so disk reads, PCIe copies, the update kernel and disk writes of three consecutive buckets overlap; device memory
holds 3 × bucket floats regardless of model size.  The updated parameters are written in the model's dtype into the
flat parameter buffer the trainer (and, colocated, the engine) reads.
"""
from __future__ import annotations

import os
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

from .. import ops

FILES = ("master", "exp_avg", "exp_avg_sq")


class NvmeStreamAdam:
    def __init__(self, flat_param: torch.Tensor, directory: str, *, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 bucket_numel: int = 64 << 20, rank: int = 0, decay_mask: torch.Tensor | None = None):
        """`flat_param`: the flat (bf16 or fp32) parameter buffer this optimizer updates in place.  `decay_mask` (fp32, same
        length, on the parameters' device): weight decay applies only where it is 1."""
        self.param = flat_param
        self.decay_mask = decay_mask
        self.n = flat_param.numel()
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.bucket = min(bucket_numel, self.n)
        self.dir = os.path.join(directory, f"rank{rank}")
        os.makedirs(self.dir, exist_ok=True)
        self.step_count = 0
        self.maps: dict[str, np.memmap] = {}
        fresh = not all(os.path.exists(self._path(k)) for k in FILES)
        for k in FILES:
            self.maps[k] = np.memmap(self._path(k), dtype=np.float32, mode="w+" if fresh else "r+", shape=(self.n,))
        if fresh:
            self._init_master()
        dev = flat_param.device
        pin = dev.type == "cuda"
        # two sets of pinned staging buffers (read-ahead / write-behind) and one set on the device
        self.host = [{k: torch.empty(self.bucket, dtype=torch.float32, pin_memory=pin) for k in FILES} for _ in range(2)]
        self.dev = {k: torch.empty(self.bucket, dtype=torch.float32, device=dev) for k in FILES} if pin else None
        self.io = ThreadPoolExecutor(max_workers=2, thread_name_prefix="nvme-adam")
        self.bytes_read = self.bytes_written = 0
        self._lock = threading.Lock()

    def _path(self, k: str) -> str:
        return os.path.join(self.dir, k + ".bin")

    def _init_master(self):
        for lo in range(0, self.n, self.bucket):
            hi = min(self.n, lo + self.bucket)
            self.maps["master"][lo:hi] = self.param[lo:hi].detach().float().cpu().numpy()
            self.maps["exp_avg"][lo:hi] = 0.0
            self.maps["exp_avg_sq"][lo:hi] = 0.0
        for m in self.maps.values():
            m.flush()

    # ---- IO (background threads) ---------------------------------------------------------------------
    def _read(self, slot: int, lo: int, hi: int):
        for k in FILES:
            self.host[slot][k][: hi - lo].copy_(torch.from_numpy(self.maps[k][lo:hi]))
        with self._lock:
            self.bytes_read += 3 * 4 * (hi - lo)

    def _write(self, slot: int, lo: int, hi: int):
        for k in FILES:
            self.maps[k][lo:hi] = self.host[slot][k][: hi - lo].numpy()
        with self._lock:
            self.bytes_written += 3 * 4 * (hi - lo)

    # ---- step ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, flat_grad: torch.Tensor, grad_scale: float = 1.0, lr: float | None = None):
        assert flat_grad.numel() == self.n
        self.step_count += 1
        b1, b2 = self.betas
        lr = self.lr if lr is None else lr
        bounds = [(lo, min(self.n, lo + self.bucket)) for lo in range(0, self.n, self.bucket)]
        pending_read = self.io.submit(self._read, 0, *bounds[0])
        pending_write = None
        for i, (lo, hi) in enumerate(bounds):
            slot = i & 1
            pending_read.result()
            if i + 1 < len(bounds):
                if pending_write is not None:          # the other slot must be flushed before it is overwritten
                    pending_write.result()
                    pending_write = None
                pending_read = self.io.submit(self._read, slot ^ 1, *bounds[i + 1])
            m = hi - lo
            h = self.host[slot]
            if self.dev is not None:
                d = {k: self.dev[k][:m] for k in FILES}
                for k in FILES:
                    d[k].copy_(h[k][:m], non_blocking=True)
            else:
                d = {k: h[k][:m] for k in FILES}
            if self.decay_mask is None:
                ops.adamw_step(d["master"], flat_grad[lo:hi], d["exp_avg"], d["exp_avg_sq"], lr=lr, beta1=b1, beta2=b2, eps=self.eps,
                               weight_decay=self.wd, step=self.step_count, grad_scale=grad_scale, param_out=self.param[lo:hi])
            elif self.dev is not None:
                ops._k().adamw_step_masked(d["master"], flat_grad[lo:hi], d["exp_avg"], d["exp_avg_sq"], self.decay_mask[lo:hi], lr, b1, b2,
                                           self.eps, self.wd, self.step_count, grad_scale, self.param[lo:hi])
            else:
                gs = flat_grad[lo:hi].float() * grad_scale
                d["exp_avg"].mul_(b1).add_(gs, alpha=1 - b1)
                d["exp_avg_sq"].mul_(b2).addcmul_(gs, gs, value=1 - b2)
                denom = (d["exp_avg_sq"] / (1 - b2 ** self.step_count)).sqrt_().add_(self.eps)
                d["master"].mul_(1 - lr * self.wd * self.decay_mask[lo:hi]).addcdiv_(d["exp_avg"] / (1 - b1 ** self.step_count), denom, value=-lr)
                self.param[lo:hi].copy_(d["master"])
            if self.dev is not None:
                for k in FILES:
                    h[k][:m].copy_(d[k], non_blocking=True)
                torch.cuda.current_stream().synchronize()
            if pending_write is not None:
                pending_write.result()
            pending_write = self.io.submit(self._write, slot, lo, hi)
        if pending_write is not None:
            pending_write.result()

    def tensor(self, key: str) -> torch.Tensor:
        """The whole state file as a CPU tensor that SHARES the mapping (reads and writes go to the file)."""
        return torch.from_numpy(self.maps[key])

    def reload_master(self):
        """Rewrite the master file from the current parameters (after loading weights); the moments stay."""
        for lo in range(0, self.n, self.bucket):
            hi = min(self.n, lo + self.bucket)
            self.maps["master"][lo:hi] = self.param[lo:hi].detach().float().cpu().numpy()

    def flush(self):
        for m in self.maps.values():
            m.flush()

    def state_dict(self) -> dict:
        self.flush()
        return {"step": self.step_count, "dir": self.dir, "numel": self.n}

    def load_state_dict(self, sd: dict):
        assert sd["numel"] == self.n
        self.step_count = sd["step"]

    def close(self):
        self.flush()
        self.io.shutdown(wait=True)
