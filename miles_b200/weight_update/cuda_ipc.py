"""Weight transfer between PROCESSES on one GPU box through CUDA IPC: the engine maps the trainer's bucket and copies out of it.

When the rollout engine runs in its own process (behind HTTP) on a GPU the trainer can reach, sending weights as bytes over
a socket would move every parameter through host memory twice.  The reference's colocated protocol instead packs a bucket of
tensors into one flat device buffer, exports an IPC handle, and posts only the handle and a manifest; the engine process opens
the handle, copies device-to-device into its parameters and acknowledges; the trainer then reuses the buffer for the next
bucket (miles/backends/training_utils/weight_update/protocols/cuda_ipc.py:34-264, the "flattened_bucket" load format of
`update_weights_from_tensor`).

    sender                                                    receiver (engine process)
    pack_bucket(named) → flat uint8 [bytes], manifest         open_bucket(blob) → flat view of the SAME memory
    export_bucket(flat, manifest) → blob (base64 text)        split → [(name, tensor view)] → copy into parameters
    POST /update_weights_from_tensor {"ipc_bucket": blob}     respond; views dropped, mapping closed
    wait for the response, then reuse `flat`

The handle is only valid while the sender keeps `flat` alive, hence the synchronous acknowledge.  On CPU tensors (tests,
engines on other hosts) the same manifest travels with the bytes themselves (`serialize_bucket`).
"""
from __future__ import annotations

import base64
import io
import pickle

import torch

ALIGN = 256


def pack_bucket(named: list[tuple[str, torch.Tensor]], out: torch.Tensor | None = None):
    """→ (flat uint8 tensor on the tensors' device, manifest [(name, dtype string, shape, offset, nbytes)]).  `out`: a reusable
    buffer at least as large as the bucket."""
    manifest, off = [], 0
    for n, t in named:
        nb = t.numel() * t.element_size()
        manifest.append((n, str(t.dtype).replace("torch.", ""), tuple(t.shape), off, nb))
        off += (nb + ALIGN - 1) // ALIGN * ALIGN
    dev = named[0][1].device if named else torch.device("cpu")
    flat = out[:off] if out is not None and out.numel() >= off else torch.empty(off, dtype=torch.uint8, device=dev)
    for (n, t), (_, _, _, o, nb) in zip(named, manifest):
        if nb:
            flat[o:o + nb].copy_(t.detach().contiguous().reshape(-1).view(torch.uint8))
    return flat, manifest


def split_bucket(flat: torch.Tensor, manifest) -> list[tuple[str, torch.Tensor]]:
    out = []
    for n, dt, shape, off, nb in manifest:
        dtype = getattr(torch, dt)
        out.append((n, flat[off:off + nb].view(dtype).reshape(shape) if nb else torch.empty(shape, dtype=dtype, device=flat.device)))
    return out


def export_bucket(flat: torch.Tensor, manifest) -> str:
    """CUDA: an IPC handle of `flat`; the caller must keep `flat` alive until the receiver has answered."""
    assert flat.is_cuda, "IPC export needs a device buffer; use serialize_bucket for host tensors"
    from torch.multiprocessing.reductions import reduce_tensor

    torch.cuda.current_stream(flat.device).synchronize()           # the packing copies must have landed before the peer reads
    fn, args = reduce_tensor(flat)
    return base64.b64encode(pickle.dumps({"kind": "ipc", "rebuild": (fn, args), "manifest": manifest})).decode()


def serialize_bucket(flat: torch.Tensor, manifest) -> str:
    buf = io.BytesIO()
    torch.save(flat.cpu(), buf)
    return base64.b64encode(pickle.dumps({"kind": "bytes", "data": buf.getvalue(), "manifest": manifest})).decode()


def open_bucket(blob: str, device) -> tuple[torch.Tensor, list]:
    """Receiver side: the flat buffer (a mapping of the sender's memory for `ipc`, a local tensor for `bytes`) + manifest."""
    d = pickle.loads(base64.b64decode(blob))
    if d["kind"] == "ipc":
        fn, args = d["rebuild"]
        flat = fn(*args)
        if device is not None and flat.device != torch.device(device):
            # the sender's buffer lives on another GPU: ONE device-to-device copy of the whole bucket over NVLink (a DMA
            # transfer, no kernel reads peer memory), then everything downstream works on local memory
            flat = flat.to(device)
        return flat, d["manifest"]
    flat = torch.load(io.BytesIO(d["data"]), map_location=device, weights_only=True)
    return flat, d["manifest"]


def send_bucket(post, named: list[tuple[str, torch.Tensor]], *, weight_version=None, staging: torch.Tensor | None = None) -> int:
    """Pack, export and post one bucket; returns its size in bytes.  `post(body_dict)` performs the request and returns once
    the receiver has copied the tensors."""
    if not named:
        return 0
    flat, manifest = pack_bucket(named, staging)
    blob = export_bucket(flat, manifest) if flat.is_cuda else serialize_bucket(flat, manifest)
    post({"ipc_bucket": blob, "weight_version": weight_version, "load_format": "flattened_bucket"})
    return int(flat.numel())
