"""LoRA adapters on the fused projections, with adapter *slots* for multi-tenant training.

What the reference gets from Megatron-Bridge PEFT plus its own slot machinery (miles/backends/megatron_utils/lora/
bridge.py:123-256, lora/model.py:21-81, lora/optimizer.py, lora/utils.py:27-72): adapters pre-wrapped around the
linear layers, the base model frozen, replicated adapter gradients all-reduced over TP, per-slot optimizers, adapter
save/export in PEFT layout, and merged weights for the rollout engine.

Layout here.  Every adapted projection `W [out, in]` owns `A [S, r, in]` and `B [S, out, r]` for S slots; one pair of
GEMMs serves all slots: `t = x·A_allᵀ` (`[T, S·r]`), rows masked to their token's slot, `Δ = t·B_all` — no per-slot
loop, no gather/scatter, and it runs through the same tensor-core GEMM as the base projection.  Under tensor
parallelism the adapter follows the base weight's split: column-parallel (wqkv, w13) keeps A replicated and shards B
by output rows; row-parallel (wo, w2) shards A by input columns and keeps B replicated.  Replicated halves carry the
suffix `_r` so the optimizer sums their gradients over the TP group.
"""
from __future__ import annotations

import contextlib
import json
import math
import os

import torch
import torch.nn as nn

from .. import ops

COLUMN, ROW = "column", "row"
_KIND = {"wqkv": COLUMN, "w13": COLUMN, "wo": ROW, "w2": ROW}


class LoRAAdapter(nn.Module):
    def __init__(self, name: str, base: torch.Tensor, full_in: int, full_out: int, rank: int, alpha: float, dropout: float,
                 slots: int, ps, seed: int):
        super().__init__()
        self.name, self.kind, self.rank, self.slots, self.ps = name, _KIND[name], rank, slots, ps
        self.scale = alpha / rank
        self.dropout = dropout
        out_local, in_local = base.shape
        gen = torch.Generator().manual_seed(seed)
        bound = 1.0 / math.sqrt(full_in)                  # kaiming-uniform(a=√5) over the full fan-in
        a_full = (torch.rand(slots, rank, full_in, generator=gen) * 2 - 1) * bound
        if self.kind == ROW and ps.tp_size > 1:
            a_full = a_full.chunk(ps.tp_size, dim=2)[ps.tp_rank]
        a = a_full.to(device=base.device, dtype=base.dtype).contiguous()
        b = torch.zeros(slots, out_local, rank, device=base.device, dtype=base.dtype)
        if self.kind == COLUMN:
            self.A_r, self.B = nn.Parameter(a), nn.Parameter(b)
        else:
            self.A, self.B_r = nn.Parameter(a), nn.Parameter(b)

    @property
    def a(self) -> torch.Tensor:
        return self.A_r if self.kind == COLUMN else self.A

    @property
    def b(self) -> torch.Tensor:
        return self.B if self.kind == COLUMN else self.B_r

    def forward(self, x: torch.Tensor, meta=None) -> torch.Tensor:
        S, r = self.slots, self.rank
        a2 = self.a.reshape(S * r, -1)
        b2 = self.b.permute(1, 0, 2).reshape(-1, S * r)
        if self.dropout > 0 and self.training:
            x = torch.nn.functional.dropout(x, self.dropout)
        slots = getattr(meta, "lora_slots", None)
        if self.kind == COLUMN:
            t = self.ps.column_linear(x, a2)              # gathers the sequence shards first under SP
        else:
            t = self.ps.row_linear(x, a2)                 # partial sums reduced (and sequence-scattered under SP)
            if slots is not None:
                slots = self.ps.sp_slice(slots)
        if slots is not None or S > 1:
            if slots is None:
                slots = torch.zeros(t.shape[0], dtype=torch.long, device=t.device)
            onehot = (slots.view(-1, 1) == torch.arange(S, device=t.device).view(1, -1)).to(t.dtype)
            t = (t.view(-1, S, r) * onehot.unsqueeze(-1)).reshape(-1, S * r)
        return ops.linear(t, b2) * self.scale

    def delta_weight(self, slot: int = 0) -> torch.Tensor:
        """scale · B[slot] · A[slot] for this rank's shard of the base weight."""
        return (self.b[slot].float() @ self.a[slot].float()) * self.scale


def _targets(model):
    for li, layer in enumerate(model.layers):
        attn = getattr(layer, "attn", None)
        if attn is not None:
            yield layer.layer, "attn", attn
        ffn = getattr(layer, "mlp", None)
        if ffn is not None and hasattr(ffn, "w13") and ffn.w13.dim() == 2:   # dense FFN only; experts stay frozen
            yield layer.layer, "ffn", ffn


def apply_lora(model, args, freeze_base: bool = True) -> list[LoRAAdapter]:
    """Attach adapters to every layer's target projections and freeze everything else."""
    cfg, ps = model.cfg, model.ps
    want = set(getattr(args, "lora_target_modules", None) or _KIND)
    unknown = want - set(_KIND)
    assert not unknown, f"unknown --lora-target-modules {sorted(unknown)} (choose from {sorted(_KIND)})"
    full_dims = {"wqkv": (cfg.hidden_size, cfg.qkv_size), "wo": (cfg.q_size, cfg.hidden_size),
                 "w13": (cfg.hidden_size, 2 * cfg.ffn_hidden_size), "w2": (cfg.ffn_hidden_size, cfg.hidden_size)}
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    out = []
    for li, where, mod in _targets(model):
        adapters = nn.ModuleDict()
        for name in ("wqkv", "wo") if where == "attn" else ("w13", "w2"):
            if name not in want:
                continue
            fin, fout = full_dims[name]
            ad = LoRAAdapter(name, getattr(mod, name), fin, fout, args.lora_rank, getattr(args, "lora_alpha", 16.0),
                             getattr(args, "lora_dropout", 0.0), getattr(args, "lora_num_slots", 1), ps,
                             seed=getattr(args, "seed", 0) * 1000003 + li * 16 + list(_KIND).index(name))
            adapters[name] = ad
            out.append(ad)
        if len(adapters):
            mod.lora = adapters
    model.lora_adapters = out
    path = getattr(args, "lora_adapter_path", None)
    if path:
        load_adapter(model, path)
    return out


def adapters_of(model) -> list[LoRAAdapter]:
    return list(getattr(model, "lora_adapters", []))


def lora_state_dict(model, slot: int | None = None) -> dict[str, torch.Tensor]:
    sd = {}
    for n, p in model.named_parameters():
        if ".lora." in n:
            sd[n] = (p.detach() if slot is None else p.detach()[slot:slot + 1]).cpu().clone()
    return sd


def load_lora_state_dict(model, sd: dict[str, torch.Tensor], slot: int | None = None):
    params = dict(model.named_parameters())
    with torch.no_grad():
        for n, t in sd.items():
            p = params[n]
            if slot is None:
                p.copy_(t.to(p))
            else:
                p[slot].copy_(t[0].to(p))


def zero_slot(model, slot: int, seed: int = 0):
    """Recycle an adapter slot for a new tenant: fresh A, zero B."""
    with torch.no_grad():
        for i, ad in enumerate(adapters_of(model)):
            gen = torch.Generator().manual_seed(seed * 7919 + i)
            bound = 1.0 / math.sqrt(ad.a.shape[-1] * (ad.ps.tp_size if ad.kind == ROW else 1))
            ad.a[slot].copy_(((torch.rand(ad.a.shape[1:], generator=gen) * 2 - 1) * bound).to(ad.a))
            ad.b[slot].zero_()


@contextlib.contextmanager
def merged(model, slot: int = 0):
    """Temporarily fold slot `slot` into the base weights (for weight sync to the engine / HF export); the exact
    original tensors are put back on exit."""
    saved = []
    with torch.no_grad():
        for li, where, mod in _targets(model):
            for name, ad in getattr(mod, "lora", {}).items():
                w = getattr(mod, name)
                saved.append((w, w.detach().clone()))
                w.add_(ad.delta_weight(slot).to(w.dtype))
    try:
        yield model
    finally:
        with torch.no_grad():
            for w, orig in saved:
                w.copy_(orig)


# ---- PEFT-layout export / import ------------------------------------------------------------------

def _full_ab(ad: LoRAAdapter, slot: int, cfg):
    """Adapter halves of the un-sharded projection (gathers the sharded half over the TP group)."""
    import torch.distributed as dist

    a, b = ad.a[slot].detach(), ad.b[slot].detach()
    ps = ad.ps
    if ps.tp_size > 1:
        if ad.kind == ROW:
            parts = [torch.empty_like(a) for _ in range(ps.tp_size)]
            dist.all_gather(parts, a.contiguous(), group=ps.tp_group)
            a = torch.cat(parts, dim=1)
        else:
            parts = [torch.empty_like(b) for _ in range(ps.tp_size)]
            dist.all_gather(parts, b.contiguous(), group=ps.tp_group)
            if ad.name == "wqkv":
                from ..models.qwen3 import unshard_qkv
                b = unshard_qkv(parts, cfg)
            else:  # w13 shards are [gate_shard; up_shard]
                g = torch.cat([p.chunk(2, 0)[0] for p in parts], 0)
                u = torch.cat([p.chunk(2, 0)[1] for p in parts], 0)
                b = torch.cat([g, u], 0)
    return a.float().cpu(), b.float().cpu()


def export_peft(model, out_dir: str, slot: int = 0, base_model_name: str = "") -> str:
    """Write `adapter_config.json` + `adapter_model.safetensors` with HF PEFT parameter names."""
    from ..checkpoint.hf_io import save_safetensors

    cfg = model.cfg
    tensors = {}
    mods = set()
    for li, where, mod in _targets(model):
        for name, ad in getattr(mod, "lora", {}).items():
            a, b = _full_ab(ad, slot, cfg)
            pre = f"base_model.model.model.layers.{li}"
            if name == "wqkv":
                bq, bk, bv = b.split([cfg.q_size, cfg.kv_size, cfg.kv_size], 0)
                for proj, bb in (("q_proj", bq), ("k_proj", bk), ("v_proj", bv)):
                    tensors[f"{pre}.self_attn.{proj}.lora_A.weight"] = a.clone()
                    tensors[f"{pre}.self_attn.{proj}.lora_B.weight"] = bb.contiguous()
                    mods.add(proj)
            elif name == "wo":
                tensors[f"{pre}.self_attn.o_proj.lora_A.weight"] = a
                tensors[f"{pre}.self_attn.o_proj.lora_B.weight"] = b
                mods.add("o_proj")
            elif name == "w13":
                bg, bu = b.chunk(2, 0)
                for proj, bb in (("gate_proj", bg), ("up_proj", bu)):
                    tensors[f"{pre}.mlp.{proj}.lora_A.weight"] = a.clone()
                    tensors[f"{pre}.mlp.{proj}.lora_B.weight"] = bb.contiguous()
                    mods.add(proj)
            else:
                tensors[f"{pre}.mlp.down_proj.lora_A.weight"] = a
                tensors[f"{pre}.mlp.down_proj.lora_B.weight"] = b
                mods.add("down_proj")
    if model.ps.rank == 0 or not torch.distributed.is_initialized():
        os.makedirs(out_dir, exist_ok=True)
        ad0 = adapters_of(model)[0]
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "r": ad0.rank, "lora_alpha": ad0.scale * ad0.rank, "lora_dropout": ad0.dropout,
                       "target_modules": sorted(mods), "base_model_name_or_path": base_model_name, "bias": "none",
                       "task_type": "CAUSAL_LM"}, f, indent=1)
        save_safetensors(os.path.join(out_dir, "adapter_model.safetensors"), tensors)
    return out_dir


def save_adapter(model, path: str, slot: int | None = None):
    """This package's own adapter file (rank-local shards; one file per rank)."""
    os.makedirs(path, exist_ok=True)
    torch.save(lora_state_dict(model, slot), os.path.join(path, f"adapter_rank{model.ps.rank}.pt"))


def load_adapter(model, path: str, slot: int | None = None):
    f = os.path.join(path, f"adapter_rank{model.ps.rank}.pt")
    load_lora_state_dict(model, torch.load(f, map_location="cpu"), slot)


# ---- per-slot optimizer -----------------------------------------------------------------------------

class SlotOptimizer:
    """AdamW state per adapter slot, so that tenants sharing one base model step independently
    (the reference's `SlotOptimizer`, miles/backends/megatron_utils/lora/optimizer.py).  Adapters are small, so this
    runs as plain tensor ops on slices `A[slot]`, `B[slot]`; gradients of TP-replicated halves are summed first."""

    def __init__(self, model, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        self.model, self.betas, self.eps, self.wd = model, betas, eps, weight_decay
        self.params = [(n, p) for n, p in model.named_parameters() if ".lora." in n]
        self.state: dict[int, dict] = {}

    def _slot_state(self, slot: int):
        if slot not in self.state:
            self.state[slot] = {"step": 0, "m": [torch.zeros_like(p[slot], dtype=torch.float32) for _, p in self.params],
                                "v": [torch.zeros_like(p[slot], dtype=torch.float32) for _, p in self.params]}
        return self.state[slot]

    def reset_slot(self, slot: int):
        self.state.pop(slot, None)

    def zero_grad(self):
        for _, p in self.params:
            p.grad = None

    @torch.no_grad()
    def step(self, slot: int, lr: float, clip_grad: float = 0.0) -> float:
        import torch.distributed as dist

        ps = self.model.ps
        grads = []
        for n, p in self.params:
            g = (p.grad[slot] if p.grad is not None else torch.zeros_like(p[slot])).float()
            if ps.tp_size > 1 and n.rsplit(".", 1)[-1].endswith("_r"):
                dist.all_reduce(g, group=ps.tp_group)
            grads.append(g)
        sq = sum((g * g).sum() for g in grads)
        if ps.tp_size > 1:
            # sharded halves contribute distinct elements per rank, replicated halves the same ones on every rank
            rep = sum((g * g).sum() for (n, _), g in zip(self.params, grads) if n.rsplit(".", 1)[-1].endswith("_r"))
            part = sq - rep
            dist.all_reduce(part, group=ps.tp_group)
            sq = part + rep
        norm = float(sq.sqrt())
        coef = min(1.0, clip_grad / (norm + 1e-6)) if clip_grad > 0 else 1.0
        st = self._slot_state(slot)
        st["step"] += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
        for (n, p), g, m, v in zip(self.params, grads, st["m"], st["v"]):
            g = g * coef
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            w = p[slot].float()
            w = w - lr * (upd + self.wd * w)
            p[slot].copy_(w.to(p.dtype))
        return norm

    def state_dict(self):
        return {"state": self.state}

    def load_state_dict(self, sd):
        self.state = sd["state"]
