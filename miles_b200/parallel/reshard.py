"""Trainer → engine weight sync across DIFFERENT parallel layouts: reshard inside the copy kernel, straight into peer memory.

The reference gathers the trainer's TP / EP shards into full HF-named tensors bucket by bucket (all-gathers), converts,
optionally quantises, and hands the buckets to the engine, which re-shards them for its own layout
(miles/backends/megatron_utils/update_weight/hf_weight_iterator_direct.py:31-476, expert_gather.py:29-164,
training_utils/weight_update/protocols/cuda_ipc.py:34-264).  On one NVSwitch box every engine buffer is addressable from
every trainer GPU, so no intermediate full tensor is needed: each trainer rank works out which RECTANGLES of its shards
land where in each engine rank's shards and one kernel per bucket stores them there (`ops/csrc/weight_sync.cu`
`multi_copy2d`: rows × row-bytes rectangles with independent source and destination pitch, optional MXFP8
quantise-dequantise of 1×32 blocks on the way).  A cross-rank flag barrier ends the transfer.

Sharding rules of this package's parameter layout (see `models/qwen3.py`), as rectangles of a 2-D view of the FULL tensor:
  attn.wqkv / attn.bqkv   [q; k; v] row blocks, each split by TP rank          (3 row blocks per rank)
  mlp.w13 (dense)          [gate; up] row blocks, each split by TP rank         (2 row blocks per rank)
  attn.wo, mlp.w2 (dense)  column band per TP rank
  lm_head                  row block per TP rank
  mlp.w13 / mlp.w2 (MoE)   [E, …] split by EP rank along the expert axis        (one row block per rank; expert-TP is 1)
  everything else          replicated
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..models.config import ModelConfig

ITEM_BYTES = 16384        # as kChunkBytes in weight_sync.cu


@dataclass(frozen=True)
class Rect:
    """`rows × cols` elements of the full 2-D view at (grow, gcol) that live at (lrow, lcol) of a rank's local 2-D view."""

    grow: int
    gcol: int
    lrow: int
    lcol: int
    rows: int
    cols: int


def _suffix(name: str) -> str:
    return name.split(".", 2)[-1] if name.startswith("layers.") else name


def full_shape_2d(name: str, local_shape: tuple, cfg: ModelConfig, tp: int, ep: int) -> tuple[int, int]:
    """(rows, cols) of the 2-D view of the full (unsharded) tensor; leading expert axes are folded into the rows."""
    sfx = _suffix(name)
    if len(local_shape) == 3:                                   # stacked experts [E_local, a, b]
        return local_shape[0] * ep * local_shape[1], local_shape[2]
    if len(local_shape) == 1:
        n = local_shape[0]
        return (n * tp if sfx.endswith("attn.bqkv") else n), 1
    r, c = local_shape
    if sfx.endswith(("attn.wqkv", "mlp.w13")) or sfx == "lm_head":
        return r * tp, c
    if sfx.endswith(("attn.wo", "mlp.w2")):
        return r, c * tp
    return r, c


def local_rects(name: str, local_shape: tuple, cfg: ModelConfig, tp: int, tp_rank: int, ep: int, ep_rank: int) -> list[Rect]:
    """Where the local tensor of (tp_rank, ep_rank) sits in the full tensor."""
    sfx = _suffix(name)
    if len(local_shape) == 3:
        e_local, a, b = local_shape
        return [Rect(ep_rank * e_local * a, 0, 0, 0, e_local * a, b)]
    if len(local_shape) == 1:
        n = local_shape[0]
        if sfx.endswith("attn.bqkv") and tp > 1:
            return _stacked_blocks([cfg.q_size, cfg.kv_size, cfg.kv_size], tp, tp_rank, 1)
        return [Rect(0, 0, 0, 0, n, 1)]
    r, c = local_shape
    if tp == 1:
        return [Rect(0, 0, 0, 0, r, c)]
    if sfx.endswith("attn.wqkv"):
        return _stacked_blocks([cfg.q_size, cfg.kv_size, cfg.kv_size], tp, tp_rank, c)
    if sfx.endswith("mlp.w13"):
        half = r * tp // 2
        return _stacked_blocks([half, half], tp, tp_rank, c)
    if sfx == "lm_head":
        return [Rect(tp_rank * r, 0, 0, 0, r, c)]
    if sfx.endswith(("attn.wo", "mlp.w2")):
        return [Rect(0, tp_rank * c, 0, 0, r, c)]
    return [Rect(0, 0, 0, 0, r, c)]


def _stacked_blocks(parts: list[int], tp: int, tp_rank: int, cols: int) -> list[Rect]:
    out, g0, l0 = [], 0, 0
    for n in parts:
        per = n // tp
        out.append(Rect(g0 + tp_rank * per, 0, l0, 0, per, cols))
        g0 += n
        l0 += per
    return out


def is_replicated(name: str, local_shape: tuple, tp: int, ep: int) -> bool:
    """True when every rank of the layout holds the whole tensor."""
    sfx = _suffix(name)
    if len(local_shape) == 3:
        return ep == 1
    if tp == 1:
        return True
    if len(local_shape) == 1:
        return not sfx.endswith("attn.bqkv")
    return not (sfx.endswith(("attn.wqkv", "mlp.w13", "attn.wo", "mlp.w2")) or sfx == "lm_head")


def intersect(a: Rect, b: Rect):
    """Overlap of two rectangles in the full view → (a-local row, a-local col, b-local row, b-local col, rows, cols) or None."""
    r0, r1 = max(a.grow, b.grow), min(a.grow + a.rows, b.grow + b.rows)
    c0, c1 = max(a.gcol, b.gcol), min(a.gcol + a.cols, b.gcol + b.cols)
    if r0 >= r1 or c0 >= c1:
        return None
    return (a.lrow + r0 - a.grow, a.lcol + c0 - a.gcol, b.lrow + r0 - b.grow, b.lcol + c0 - b.gcol, r1 - r0, c1 - c0)


def plan_copies(name: str, src_shape: tuple, dst_shape: tuple, cfg: ModelConfig, src: tuple[int, int, int, int],
                dst: tuple[int, int, int, int]) -> list[tuple[int, int, int, int, int, int]]:
    """Rectangles to copy from the shard of source coordinates `src` = (tp, tp_rank, ep, ep_rank) into the shard of
    destination coordinates `dst`, as (src row, src col, dst row, dst col, rows, cols) of the two local 2-D views."""
    out = []
    for a in local_rects(name, src_shape, cfg, *src):
        for b in local_rects(name, dst_shape, cfg, *dst):
            hit = intersect(a, b)
            if hit is not None:
                out.append(hit)
    return out


def local_2d(shape: tuple) -> tuple[int, int]:
    if len(shape) == 3:
        return shape[0] * shape[1], shape[2]
    if len(shape) == 1:
        return shape[0], 1
    return shape[0], shape[1]


class ReshardPlan:
    """One trainer rank's part of a trainer → engines transfer over the NVLink fabric.

    Collective construction (every rank of the box, same order): the engine's parameters are re-homed into one symmetric
    buffer so that every trainer rank can address every engine rank's shards; then each rank lists its rectangles.
    Senders: a destination engine rank takes TP-sharded tensors from the trainer ranks of ITS tensor-parallel group, expert
    tensors from its expert-parallel group, and replicated tensors from the trainer rank on its own GPU — so every byte is
    sent once and, where layouts coincide, never leaves the GPU."""

    def __init__(self, actor, engine, fab, quant: str | None = None):
        self.actor, self.engine, self.fab, self.quant = actor, engine, fab, quant
        ps_t, ps_e = actor.ps, engine.ps
        cfg = actor.cfg
        self.world = ps_t.world_size
        e_named = list(engine.model.named_parameters())
        # ---- engine parameters → one symmetric allocation (same layout on every rank: engines are replicas of one layout)
        offs, total = {}, 0
        for n, p in e_named:
            offs[n] = total
            total += (p.numel() * p.element_size() + 255) // 256 * 256
        flat = fab.alloc(total, torch.uint8, "engine.params")
        with torch.no_grad():
            for n, p in e_named:
                nb = p.numel() * p.element_size()
                view = flat[offs[n]:offs[n] + nb].view(p.dtype).view(p.shape)
                view.copy_(p.data)
                p.data = view
        sym, base = fab.sym_of(flat)
        e_shapes = {n: tuple(p.shape) for n, p in e_named}
        t_named = dict(actor.model.named_parameters())
        me = ps_t.rank
        t_coord = (ps_t.tp_size, ps_t.tp_rank, ps_t.ep_size, ps_t.ep_rank)
        tp_e, ep_e = ps_e.tp_size, ps_e.ep_size
        rows: list[tuple] = []
        self.bytes = 0
        for d in range(self.world):
            # engine coordinates of rank d follow the same rank order as the trainer's groups (tp fastest, ep over the block)
            d_tp_rank = d % tp_e
            d_ep_rank = d % ep_e if ep_e > 1 else 0
            d_coord = (tp_e, d_tp_rank, ep_e, d_ep_rank)
            same_tp_group = (d // ps_t.tp_size) == (me // ps_t.tp_size)
            same_ep_group = (d // ps_t.ep_size) == (me // ps_t.ep_size)
            dst_base = sym.views[d].data_ptr() + base
            for n, p in t_named.items():
                if n not in e_shapes or ".lora." in n or ".value_head." in n:
                    continue
                ts = tuple(p.shape)
                expert = len(ts) == 3
                if is_replicated(n, ts, ps_t.tp_size, ps_t.ep_size):
                    if d != me:
                        continue                              # the trainer rank on the engine's own GPU sends replicated tensors
                elif not (same_ep_group if expert else same_tp_group):
                    continue
                esz = p.element_size()
                _, sc = local_2d(ts)
                _, dc = local_2d(e_shapes[n])
                for (sr, scol, dr, dcol, nr, ncol) in plan_copies(n, ts, e_shapes[n], cfg, t_coord, d_coord):
                    src_ptr = p.data_ptr() + (sr * sc + scol) * esz
                    dst_ptr = dst_base + offs[n] + (dr * dc + dcol) * esz
                    if ncol == sc and ncol == dc:             # whole rows on both sides: one long row copies fastest
                        rows.append((src_ptr, dst_ptr, 1, nr * ncol * esz, nr * ncol * esz, nr * ncol * esz, n))
                    else:
                        rows.append((src_ptr, dst_ptr, nr, ncol * esz, sc * esz, dc * esz, n))
                    self.bytes += nr * ncol * esz
        self.rows = rows
        self._tables = None

    def _build_tables(self):
        from .weight_sync import _skip_quant

        dev = self.actor.device
        plain, qdq = [], []
        named = dict(self.actor.model.named_parameters())
        for r in self.rows:
            p = named[r[6]]
            want_q = self.quant in ("mxfp8", "mxfp8_qdq") and p.dtype == torch.bfloat16 and not _skip_quant(r[6], p) and r[3] % 64 == 0
            (qdq if want_q else plain).append(r[:6])
        out = []
        for rows, q in ((plain, False), (qdq, True)):
            if not rows:
                continue
            # long single-row rectangles are cut into 16 KB items by the prefix table as well
            split = []
            for (s, d, nr, rb, sp, dp) in rows:
                if nr == 1 and rb > ITEM_BYTES:
                    whole, tail = rb // ITEM_BYTES, rb % ITEM_BYTES
                    if whole:
                        split.append((s, d, whole, ITEM_BYTES, ITEM_BYTES, ITEM_BYTES))
                    if tail:
                        split.append((s + whole * ITEM_BYTES, d + whole * ITEM_BYTES, 1, tail, tail, tail))
                else:
                    split.append((s, d, nr, rb, sp, dp))
            pref, tot = [0], 0
            for (_, _, nr, rb, _, _) in split:
                rpi = max(1, ITEM_BYTES // max(rb, 1))
                tot += (nr + rpi - 1) // rpi
                pref.append(tot)
            table = torch.tensor(split, dtype=torch.int64).to(dev)
            prefix = torch.tensor(pref, dtype=torch.int64).to(dev)
            out.append((table, prefix, tot, q))
        self._tables = out

    def run(self) -> int:
        """Enqueue the transfer on the current stream and close it with a cross-rank barrier; returns bytes this rank wrote."""
        from .fabric import CH_SYNC

        if self._tables is None:
            self._build_tables()              # addresses are stable (flat trainer buffers, symmetric engine buffer): built once
        C = self.fab.C
        for table, prefix, tot, q in self._tables:
            C.multi_copy2d(table, prefix, tot, q)
        self.fab.barrier(list(range(self.world)), CH_SYNC)
        return self.bytes
