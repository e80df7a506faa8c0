"""Sharded `torch_dist` checkpoints: every rank writes and reads only its own rectangles of each Megatron-named tensor.

The reference's Megatron backend saves `iter_XXXXXXX/` as a `torch_dist` store: each parameter is one entry named as in
Megatron-core (`decoder.layers.3.self_attention.linear_qkv.weight`, experts as `…linear_fc1.weight<e>`), stored as
chunks written by the ranks that own them; the distributed optimizer's fp32 master weights and Adam moments are stored
in MODEL space under `optimizer.state.{fp32_param,exp_avg,exp_avg_sq}.<parameter name>`, so a run may resume under any
other parallel layout (miles/backends/megatron_utils/checkpoint.py:107-299, model.py:703-748;
tools/convert_torch_dist_to_hf.py:45-103 reads such a store).

Here that store is produced without DTensor, ShardedTensor or extra process groups: a small DCP planner turns each
local shard into write items — rectangles (offsets + sizes) of the full tensor — and on load asks DCP for exactly the
rectangles this rank holds, whatever partition the writer used.  The layout rules:

  attn.wqkv / bqkv   local [q_t; k_t; v_t] → Megatron's per-KV-group interleave of the LOCAL heads, one row block at
                     tp_rank · rows (the full tensor is the concatenation of the ranks' blocks, as in Megatron)
  mlp.w13 (dense)    [gate_t; up_t] → two row blocks of the full [gate; up]
  attn.wo, mlp.w2    column band
  lm_head            row block
  experts            one entry per GLOBAL expert id, written whole by the EP rank that owns it
  everything else    replicated: written once

Each chunk has exactly one writer: dense tensors by the data- and context-parallel rank 0 (replicated ones by TP rank 0
too), experts by the expert-data-parallel rank 0, tied embeddings by the first pipeline stage.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.convert import megatron_name_map, megatron_qkv_to_ours, ours_qkv_to_megatron

COMMON = "common.pt"


@dataclass
class Piece:
    """`local[rows, cols]` ↔ the rectangle of the full tensor starting at `offsets`."""

    offsets: tuple[int, ...]
    index: tuple                      # slices (or an int for the expert axis) into the local (Megatron-ordered) tensor


@dataclass
class Entry:
    key: str
    global_shape: tuple[int, ...]
    pieces: list[Piece]
    writer: bool                      # this rank writes the pieces
    qkv: bool = False                 # local tensor needs the q/k/v ↔ per-group interleave conversion


def _local_cfg(cfg: ModelConfig, tp: int) -> ModelConfig:
    assert cfg.num_kv_heads % tp == 0, "the Megatron qkv layout needs kv heads divisible by tp"
    return dataclasses.replace(cfg, num_heads=cfg.num_heads // tp, num_kv_heads=cfg.num_kv_heads // tp)


def supported(cfg: ModelConfig, ps) -> bool:
    return ps is None or ps.tp_size == 1 or cfg.num_kv_heads % ps.tp_size == 0


def entries_for(name: str, shape: tuple, cfg: ModelConfig, ps, names: dict[str, str]) -> list[Entry]:
    """Megatron entries covered by the local tensor `name` of `shape` on this rank."""
    tp, tr = (ps.tp_size, ps.tp_rank) if ps else (1, 0)
    ep, er = (ps.ep_size, ps.ep_rank) if ps else (1, 0)
    dense_writer = ps is None or (ps.dp_rank == 0 and ps.cp_rank == 0)
    key = names.get(name, f"extra.{name}")
    last = name.rsplit(".", 1)[-1]
    full = slice(None)
    if len(shape) == 3 and last in ("w13", "w2"):                       # stacked experts [E_local, a, b]
        writer = ps is None or ps.edp_rank == 0
        return [Entry(f"{key}{er * shape[0] + e}", tuple(shape[1:]), [Piece((0, 0), (e,))], writer)
                for e in range(shape[0])]
    if name == "embed" and ps is not None and not ps.is_pp_first:    # tied copy on the last stage
        return []
    if tp > 1 and last in ("wqkv", "bqkv"):
        rows = shape[0]
        g = (rows * tp,) + tuple(shape[1:])
        return [Entry(key, g, [Piece((tr * rows,) + (0,) * (len(shape) - 1), (full,))], dense_writer, qkv=True)]
    if last in ("wqkv", "bqkv"):
        return [Entry(key, tuple(shape), [Piece((0,) * len(shape), (full,))], dense_writer, qkv=True)]
    if tp > 1 and last == "w13" and len(shape) == 2:
        h = shape[0] // 2
        return [Entry(key, (shape[0] * tp, shape[1]),
                      [Piece((tr * h, 0), (slice(0, h),)), Piece((h * tp + tr * h, 0), (slice(h, 2 * h),))], dense_writer)]
    if tp > 1 and last in ("wo", "w2") and len(shape) == 2:
        return [Entry(key, (shape[0], shape[1] * tp), [Piece((0, tr * shape[1]), (full,))], dense_writer)]
    if tp > 1 and last == "lm_head":
        return [Entry(key, (shape[0] * tp, shape[1]), [Piece((tr * shape[0], 0), (full,))], dense_writer)]
    return [Entry(key, tuple(shape), [Piece((0,) * len(shape), (full,))], dense_writer and tr == 0)]


class _Chunks:
    """State-dict leaf: rectangles of one full tensor held by this rank."""

    def __init__(self, global_shape, dtype):
        self.global_shape = torch.Size(global_shape)
        self.dtype = dtype
        self.parts: list[tuple[torch.Size, torch.Tensor]] = []

    def add(self, offsets, tensor):
        self.parts.append((torch.Size(offsets), tensor))


def _planners():
    from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
    from torch.distributed.checkpoint.metadata import (ChunkStorageMetadata, MetadataIndex, TensorProperties,
                                                       TensorStorageMetadata)
    from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
    from torch.distributed.checkpoint.planner_helpers import _create_write_items, create_read_items_for_chunk_list

    class Save(DefaultSavePlanner):
        def create_local_plan(self):
            items = []
            for fqn, obj in self.state_dict.items():
                if isinstance(obj, _Chunks):
                    for off, t in obj.parts:
                        items.append(WriteItem(
                            index=MetadataIndex(fqn, off), type=WriteItemType.SHARD,
                            tensor_data=TensorWriteData(chunk=ChunkStorageMetadata(offsets=off, sizes=t.size()),
                                                        properties=TensorProperties(dtype=obj.dtype), size=obj.global_shape)))
                else:
                    items += _create_write_items(fqn, obj)
            self.plan = SavePlan(items, planner_data=getattr(self, "mappings", None) or {k: (k,) for k in self.state_dict})
            return self.plan

        def lookup_object(self, index):
            obj = self.state_dict[index.fqn]
            if isinstance(obj, _Chunks):
                for off, t in obj.parts:
                    if off == index.offset:
                        return t
                raise KeyError(index)
            return super().lookup_object(index)

    class Load(DefaultLoadPlanner):
        def set_up_planner(self, state_dict, metadata=None, is_coordinator=False):
            # the default set-up rewrites leaves it does not know; the chunk lists are kept as they are
            self.original_state_dict = self.state_dict = state_dict
            self.mappings = {k: (k,) for k in state_dict}
            self.metadata, self.is_coordinator = metadata, is_coordinator

        def finish_plan(self, plan):
            return plan

        def create_local_plan(self):
            reqs = []
            for fqn, obj in self.state_dict.items():
                md = self.metadata.state_dict_metadata.get(fqn)
                if md is None:
                    raise KeyError(f"checkpoint has no entry {fqn}")
                if isinstance(obj, _Chunks):
                    assert isinstance(md, TensorStorageMetadata) and md.size == obj.global_shape, \
                        f"{fqn}: checkpoint holds {tuple(md.size)}, the model wants {tuple(obj.global_shape)}"
                    local = [ChunkStorageMetadata(offsets=off, sizes=t.size()) for off, t in obj.parts]
                    reqs += create_read_items_for_chunk_list(fqn, md, local)
                else:
                    raise TypeError(f"{fqn}: only chunked entries are read here, got {type(obj)}")
            return LoadPlan(reqs)

        def lookup_tensor(self, index):
            obj = self.state_dict[index.fqn]
            for i, (off, t) in enumerate(obj.parts):
                if (index.offset is not None and off == index.offset) or (index.offset is None and index.index == i):
                    return t
            raise KeyError(index)

    return Save, Load


# ---- what a rank holds ---------------------------------------------------------------------------------------------

def _model_items(actor):
    return [(n, p.data) for n, p in actor.model.named_parameters_global()]


def _optimizer_items(actor, attr: str, gather: bool):
    """→ (items, flats): items are (global parameter name, fp32 view of the parameter's local shape) into one flat fp32
    buffer per reduction domain; flats lists (domain, buffer).  With `gather` the ZeRO shards of the reduction group are
    all-gathered into the buffer first (collective); without it the buffer is zero, to be filled by a load."""
    items, flats = [], []
    for d in actor.optimizer.domains:
        shard = getattr(d, attr)
        flat = torch.zeros(d.numel, dtype=torch.float32, device=shard.device)
        if gather and d.group_size > 1:
            dist.all_gather(list(flat.chunk(d.group_size)), shard.float().contiguous(), group=d.group)
        elif gather:
            flat.copy_(shard)
        flats.append((d, flat))
        for n, p, o in zip(d.names, d.params, d.offsets):
            items.append((actor.model.global_name(n), flat[o:o + p.numel()].view(p.shape)))
    return items, flats


def _build_state(named, cfg, ps, names, prefix: str, for_load: bool):
    """→ ({key: _Chunks}, [finish callbacks]).  For a load the qkv entries read into scratch and convert afterwards."""
    tp = ps.tp_size if ps else 1
    lcfg = _local_cfg(cfg, tp) if tp > 1 else cfg
    state: dict[str, _Chunks] = {}
    finish = []
    for item in named:
        name, local = item[0], item[1]
        for ent in entries_for(name, tuple(local.shape), cfg, ps, names):
            if not for_load and not ent.writer:
                continue
            src = local
            if ent.qkv:
                if for_load:
                    src = torch.empty_like(local)
                    finish.append((local, src, lcfg))
                else:
                    src = ours_qkv_to_megatron(local, lcfg)
            ch = state.setdefault(prefix + ent.key, _Chunks(ent.global_shape, local.dtype))
            for pc in ent.pieces:
                view = src[pc.index]
                ch.add(pc.offsets, view if for_load else view.detach())
    return state, finish


# ---- public ----------------------------------------------------------------------------------------------------------

def save(actor, directory: str, *, with_optimizer: bool = True, common: dict | None = None) -> None:
    """Collective: write this rank's chunks of the model (and optimizer) into the DCP store at `directory`."""
    write_staged(stage(actor, with_optimizer=with_optimizer, to_host=False), directory, common=common)


def stage(actor, *, with_optimizer: bool = True, to_host: bool = True) -> dict:
    """Collective (the optimizer shards are gathered): this rank's chunks, copied to host memory when `to_host` so that
    training may go on while another thread writes them."""
    cfg, ps = actor.cfg, actor.ps
    names = megatron_name_map(cfg)
    state, _ = _build_state(_model_items(actor), cfg, ps, names, "", for_load=False)
    if with_optimizer and hasattr(actor.optimizer, "domains"):
        for attr, label in (("master", "fp32_param"), ("exp_avg", "exp_avg"), ("exp_avg_sq", "exp_avg_sq")):
            items, flats = _optimizer_items(actor, attr, gather=True)
            st, _ = _build_state(items, cfg, ps, names, f"optimizer.state.{label}.", for_load=False)
            # the gathered flat buffer would stay alive through the views: stage the written pieces on the host instead
            for ch in st.values():
                ch.parts = [(off, t.cpu()) for off, t in ch.parts]
            state.update(st)
            del items, flats
    if to_host:
        for ch in state.values():
            ch.parts = [(off, t.cpu().clone() if t.device.type == "cpu" else t.cpu()) for off, t in ch.parts]
    return state


def write_staged(state: dict, directory: str, *, common: dict | None = None, process_group=None) -> None:
    """Collective over `process_group` (default: the world): plan and write the staged chunks."""
    import torch.distributed.checkpoint as dcp

    Save, _ = _planners()
    world = dist.is_initialized() and dist.get_world_size() > 1
    os.makedirs(directory, exist_ok=True)
    dcp.save(state, storage_writer=dcp.FileSystemWriter(directory, single_file_per_rank=True, thread_count=1),
             planner=Save(), no_dist=not world, process_group=process_group if world else None)
    if (not dist.is_initialized() or dist.get_rank() == 0) and common is not None:
        torch.save(common, os.path.join(directory, COMMON))


def has_optimizer(directory: str) -> bool:
    import torch.distributed.checkpoint as dcp

    md = dcp.FileSystemReader(directory).read_metadata()
    return any(k.startswith("optimizer.state.exp_avg.") for k in md.state_dict_metadata)


def _reader_and_prefix(directory: str):
    import torch.distributed.checkpoint as dcp

    have = dcp.FileSystemReader(directory).read_metadata().state_dict_metadata
    prefix = "model." if "embedding.word_embeddings.weight" not in have and "model.embedding.word_embeddings.weight" in have else ""
    return have, prefix


def _read(actor, directory, named, prefix, have):
    import torch.distributed.checkpoint as dcp

    _, Load = _planners()
    state, finish = _build_state(named, actor.cfg, actor.ps, megatron_name_map(actor.cfg), prefix, for_load=True)
    state = {k: v for k, v in state.items() if k in have or ".extra." not in "." + k}   # extras are optional
    dcp.load(state, storage_reader=dcp.FileSystemReader(directory), planner=Load(), no_dist=True)
    for dst, scratch, lcfg in finish:
        dst.copy_(megatron_qkv_to_ours(scratch, lcfg))


def load(actor, directory: str, *, with_optimizer: bool = True) -> dict | None:
    """Read exactly this rank's rectangles of every model entry (and of the optimizer state); returns the common state
    (None if the store has none).  The store may have been written under any parallel layout, by this package or by
    Megatron-core with per-layer entry names."""
    have, prefix = _reader_and_prefix(directory)
    _read(actor, directory, _model_items(actor), prefix, have)
    if with_optimizer and has_optimizer(directory) and hasattr(actor.optimizer, "domains"):
        load_optimizer(actor, directory)
    path = os.path.join(directory, COMMON)
    return torch.load(path, map_location="cpu", weights_only=False) if os.path.exists(path) else None


def load_optimizer(actor, directory: str) -> None:
    have, _ = _reader_and_prefix(directory)
    for attr, label in (("master", "fp32_param"), ("exp_avg", "exp_avg"), ("exp_avg_sq", "exp_avg_sq")):
        items, flats = _optimizer_items(actor, attr, gather=False)
        _read(actor, directory, items, f"optimizer.state.{label}.", have)
        for d, flat in flats:
            getattr(d, attr).copy_(flat[d.shard[0]:d.shard[1]])
