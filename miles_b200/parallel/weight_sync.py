"""Fused trainer → engine weight sync for colocated engines that keep their own buffers.

The reference moves weights to a colocated SGLang as CUDA-IPC handles of flattened buckets that the engine then copies
parameter by parameter (weight_update/protocols/cuda_ipc.py:34-264), after gathering TP/EP shards and optionally
quantising them (hf_weight_iterator_direct.py:31-476, processors/quantizer_mxfp8.py).  When trainer and engine use the
same parallel layout (the colocated default) no gather or rename is needed: parameter `p` of trainer rank r is
parameter `p` of engine rank r.  Then the whole sync is a table of (src, dst, bytes) per bucket and ONE kernel launch
per bucket (`ops/csrc/weight_sync.cu`), storing straight into the engine's buffers — on the same GPU, or on a peer GPU
through an IPC mapping (`dst_ptrs`), where the stores cross NVLink.  With `quant="mxfp8"` the same pass quantises
1×32 blocks on the way (engine buffers then hold e4m3 payload + e8m0 scales); `quant="mxfp8_qdq"` writes bf16 values
that went through MXFP8, for engines that serve bf16 but must see the quantised model's numerics.

CPU tensors (tests, gloo runs) take the plain `copy_` path with the same bucketing.
"""
from __future__ import annotations

import torch

COPY_CHUNK = 16384        # bytes per work item, as in weight_sync.cu
QUANT_CHUNK = 256 * 32    # elements per work item

# substrings of parameters that stay bf16 under MXFP8 (norms, router, embeddings, head): the reference's skip list
# (miles/utils/mxfp8.py:7-20)
MXFP8_SKIP = ("ln1", "ln2", "norm", "router", "embed", "lm_head", "bqkv", "value_head", "lora")


def _skip_quant(name: str, p: torch.Tensor) -> bool:
    # 1×32 blocks run along the last dimension and must not straddle rows
    return p.dim() < 2 or p.shape[-1] % 32 != 0 or any(s in name for s in MXFP8_SKIP)


def _buckets(pairs, bucket_bytes):
    cur, size = [], 0
    for item in pairs:
        nb = item[1].numel() * item[1].element_size()
        if cur and size + nb > bucket_bytes:
            yield cur
            cur, size = [], 0
        cur.append(item)
        size += nb
    if cur:
        yield cur


def _launch(C, rows, chunk, kind, qdq=False):
    """rows: list of (src_ptr, dst_ptr, n, aux_ptr).  Builds the device table and launches one kernel."""
    dev = torch.cuda.current_device()
    pref, tot = [0], 0
    for _, _, n, _ in rows:
        tot += (n + chunk - 1) // chunk
        pref.append(tot)
    table = torch.tensor(rows, dtype=torch.int64).to(f"cuda:{dev}", non_blocking=True)
    prefix = torch.tensor(pref, dtype=torch.int64).to(f"cuda:{dev}", non_blocking=True)
    if kind == "copy":
        C.multi_copy(table, prefix, tot)
    else:
        C.multi_mxfp8(table, prefix, tot, qdq)
    return table, prefix        # kept alive by the caller until the stream is synchronised


def fused_weight_sync(actor, engine, quant: str | None = None, bucket_bytes: int | None = None,
                      dst_ptrs: dict[str, int] | None = None) -> int:
    """Copy every trainer parameter into the engine's parameter of the same name.  Returns bytes written.

    `dst_ptrs` (name → device address) overrides the destination, e.g. addresses of a peer GPU's engine buffers that
    were opened through the fabric; `engine.quant_buffers` (name → (payload uint8 tensor, scales uint8 tensor)) receives
    the MXFP8 form when `quant == "mxfp8"`.
    """
    src = dict(actor.model.named_parameters())
    dst = dict(engine.model.named_parameters())
    missing = [n for n in src if n not in dst and ".lora." not in n and ".value_head." not in n]
    assert not missing, f"engine model lacks parameters {missing[:3]}…: layouts differ, use the tensor protocol"
    bucket_bytes = bucket_bytes or getattr(actor.args, "update_weight_buffer_size", 512 << 20)
    pairs = [(n, p) for n, p in src.items() if n in dst]
    total = 0
    if not pairs:
        return 0
    on_gpu = pairs[0][1].is_cuda
    if not on_gpu:
        with torch.no_grad():
            for n, p in pairs:
                q = p.detach()
                if quant in ("mxfp8", "mxfp8_qdq") and not _skip_quant(n, p):
                    from ..ops import reference as ref
                    payload, scales = ref.mxfp8_quant(q)
                    q = ref.mxfp8_dequant(payload, scales).reshape(q.shape).to(p.dtype)
                dst[n].copy_(q)
                total += p.numel() * p.element_size()
        return total

    from ..ops import cuda as K

    keep = []
    with torch.no_grad():
        for bucket in _buckets(pairs, bucket_bytes):
            copies, quants = [], []
            for n, p in bucket:
                d = dst[n]
                assert d.shape == p.shape and d.is_contiguous() and p.is_contiguous(), f"layout mismatch for {n}"
                dptr = dst_ptrs[n] if dst_ptrs is not None else d.data_ptr()
                nbytes = p.numel() * p.element_size()
                if quant in ("mxfp8", "mxfp8_qdq") and not _skip_quant(n, p) and p.dtype == torch.bfloat16:
                    if quant == "mxfp8" and n not in getattr(engine, "quant_buffers", {}):
                        if p.data_ptr() != dptr:            # not served in MXFP8 (e.g. stacked expert weights): plain copy
                            copies.append((p.data_ptr(), dptr, nbytes, 0))
                            total += nbytes
                        continue
                    if quant == "mxfp8":
                        payload, scales = engine.quant_buffers[n]
                        quants.append((p.data_ptr(), payload.data_ptr(), p.numel(), scales.data_ptr()))
                        total += p.numel() + p.numel() // 32
                    else:
                        quants.append((p.data_ptr(), dptr, p.numel(), 0))
                        total += nbytes
                elif p.data_ptr() != dptr:                 # aliased tensors (engine built on the trainer's model) need no copy
                    assert d.dtype == p.dtype, f"dtype mismatch for {n}"
                    copies.append((p.data_ptr(), dptr, nbytes, 0))
                    total += nbytes
            if copies:
                keep.append(_launch(K.C, copies, COPY_CHUNK, "copy"))
            if quants:
                keep.append(_launch(K.C, quants, QUANT_CHUNK, "mxfp8", qdq=(quant == "mxfp8_qdq")))
    torch.cuda.current_stream().synchronize()
    del keep
    return total
