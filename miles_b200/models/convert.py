"""Tensor-name and layout conversion: this package ⇄ Hugging Face ⇄ Megatron.

HF names are the wire/disk contract (safetensors export, weight sync to HTTP engines); Megatron names
and the grouped QKV interleave are needed to read and write Megatron `torch_dist` checkpoints.  The
mapping reproduces the reference's converters (miles/backends/megatron_utils/megatron_to_hf/qwen2.py:5-75,
qwen3moe.py:6-117): QKV is stored by Megatron as `[groups, q_per_group + 2, head_dim, hidden]`,
gate/up are stacked in `linear_fc1`, experts are named by global expert id.
"""
from __future__ import annotations

import re
from typing import Iterable, Iterator

import torch

from .config import ModelConfig


# ---- ours → HF -------------------------------------------------------------------------------

def to_hf(name: str, tensor: torch.Tensor, cfg: ModelConfig, *, expert_offset: int = 0, _plain: bool = False
          ) -> list[tuple[str, torch.Tensor]]:
    """Convert one *full* (un-sharded along TP) tensor of this package's layout into HF tensors."""
    if not _plain and getattr(cfg, "family", "qwen3") != "qwen3":
        from . import bridges           # latent / linear attention, shared experts, … of the other families

        return bridges.to_hf(name, tensor, cfg, expert_offset=expert_offset)
    if name == "embed":
        return [("model.embed_tokens.weight", tensor)]
    if name == "lm_head":
        return [("lm_head.weight", tensor)]
    if name == "norm":
        return [("model.norm.weight", tensor)]
    m = re.match(r"layers\.(\d+)\.(.+)", name)
    assert m, f"unknown parameter {name}"
    L = int(m.group(1))
    rest = m.group(2)
    pre = f"model.layers.{L}"
    if rest == "ln1":
        return [(f"{pre}.input_layernorm.weight", tensor)]
    if rest == "ln2":
        return [(f"{pre}.post_attention_layernorm.weight", tensor)]
    if rest == "attn.wqkv":
        q, k, v = tensor.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
        return [(f"{pre}.self_attn.q_proj.weight", q), (f"{pre}.self_attn.k_proj.weight", k),
                (f"{pre}.self_attn.v_proj.weight", v)]
    if rest == "attn.bqkv":
        q, k, v = tensor.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
        return [(f"{pre}.self_attn.q_proj.bias", q), (f"{pre}.self_attn.k_proj.bias", k),
                (f"{pre}.self_attn.v_proj.bias", v)]
    if rest == "attn.wo":
        return [(f"{pre}.self_attn.o_proj.weight", tensor)]
    if rest == "attn.q_norm":
        return [(f"{pre}.self_attn.q_norm.weight", tensor)]
    if rest == "attn.k_norm":
        return [(f"{pre}.self_attn.k_norm.weight", tensor)]
    if rest == "mlp.router":
        return [(f"{pre}.mlp.gate.weight", tensor)]
    if rest == "mlp.w13":
        if tensor.dim() == 3:  # experts [E_local, 2F, H]
            out = []
            for e in range(tensor.shape[0]):
                g, u = tensor[e].chunk(2, dim=0)
                ge = e + expert_offset
                out += [(f"{pre}.mlp.experts.{ge}.gate_proj.weight", g), (f"{pre}.mlp.experts.{ge}.up_proj.weight", u)]
            return out
        g, u = tensor.chunk(2, dim=0)
        return [(f"{pre}.mlp.gate_proj.weight", g), (f"{pre}.mlp.up_proj.weight", u)]
    if rest == "mlp.w2":
        if tensor.dim() == 3:
            return [(f"{pre}.mlp.experts.{e + expert_offset}.down_proj.weight", tensor[e]) for e in range(tensor.shape[0])]
        return [(f"{pre}.mlp.down_proj.weight", tensor)]
    raise KeyError(f"no HF mapping for {name}")


def hf_state_to_ours(hf: dict[str, torch.Tensor], cfg: ModelConfig, _plain: bool = False) -> dict[str, torch.Tensor]:
    """Assemble full tensors of this package's layout from an HF state dict."""
    if not _plain and getattr(cfg, "family", "qwen3") != "qwen3":
        from . import bridges

        return bridges.from_hf(hf, cfg)
    out: dict[str, torch.Tensor] = {}
    out["embed"] = hf["model.embed_tokens.weight"]
    if "lm_head.weight" in hf and not cfg.tie_embeddings:
        out["lm_head"] = hf["lm_head.weight"]
    out["norm"] = hf["model.norm.weight"]
    for L in range(cfg.num_layers):
        pre, o = f"model.layers.{L}", f"layers.{L}"
        if f"{pre}.input_layernorm.weight" not in hf:
            continue
        out[f"{o}.ln1"] = hf[f"{pre}.input_layernorm.weight"]
        out[f"{o}.ln2"] = hf[f"{pre}.post_attention_layernorm.weight"]
        if f"{pre}.self_attn.k_proj.weight" in hf:          # absent for latent / linear attention layers of other families
            out[f"{o}.attn.wqkv"] = torch.cat([hf[f"{pre}.self_attn.{x}_proj.weight"] for x in "qkv"], 0)
            if cfg.qkv_bias:
                out[f"{o}.attn.bqkv"] = torch.cat([hf[f"{pre}.self_attn.{x}_proj.bias"] for x in "qkv"], 0)
        if f"{pre}.self_attn.o_proj.weight" in hf:
            out[f"{o}.attn.wo"] = hf[f"{pre}.self_attn.o_proj.weight"]
        if cfg.qk_norm and f"{pre}.self_attn.q_norm.weight" in hf:
            out[f"{o}.attn.q_norm"] = hf[f"{pre}.self_attn.q_norm.weight"]
            out[f"{o}.attn.k_norm"] = hf[f"{pre}.self_attn.k_norm.weight"]
        if cfg.layer_is_moe(L):
            out[f"{o}.mlp.router"] = hf[f"{pre}.mlp.gate.weight"]
            out[f"{o}.mlp.w13"] = torch.stack([
                torch.cat([hf[f"{pre}.mlp.experts.{e}.gate_proj.weight"], hf[f"{pre}.mlp.experts.{e}.up_proj.weight"]], 0)
                for e in range(cfg.num_experts)])
            out[f"{o}.mlp.w2"] = torch.stack([hf[f"{pre}.mlp.experts.{e}.down_proj.weight"] for e in range(cfg.num_experts)])
        else:
            out[f"{o}.mlp.w13"] = torch.cat([hf[f"{pre}.mlp.gate_proj.weight"], hf[f"{pre}.mlp.up_proj.weight"]], 0)
            out[f"{o}.mlp.w2"] = hf[f"{pre}.mlp.down_proj.weight"]
    return out


# ---- sharding of full tensors ------------------------------------------------------------------

def shard_for_rank(name: str, full: torch.Tensor, cfg: ModelConfig, ps) -> torch.Tensor:
    """Slice a full tensor (our layout) to what rank `ps` holds under TP / EP."""
    tp, tr = ps.tp_size, ps.tp_rank
    last = name.rsplit(".", 1)[-1]
    if last in ("wqkv", "bqkv") and tp > 1:
        from .qwen3 import shard_qkv
        return shard_qkv(full, cfg, tr, tp)
    if last == "wo" and tp > 1:
        return full.chunk(tp, dim=1)[tr].contiguous()
    if last == "lm_head" and tp > 1:
        return full.chunk(tp, dim=0)[tr].contiguous()
    if last == "w13":
        if full.dim() == 3:
            e = full.shape[0] // ps.ep_size if full.shape[0] == cfg.num_experts else full.shape[0]
            return full[ps.ep_rank * e:(ps.ep_rank + 1) * e] if full.shape[0] == cfg.num_experts else full
        if tp > 1:
            g, u = full.chunk(2, dim=0)
            return torch.cat([g.chunk(tp, 0)[tr], u.chunk(tp, 0)[tr]], 0).contiguous()
    if last == "w2":
        if full.dim() == 3:
            e = full.shape[0] // ps.ep_size
            return full[ps.ep_rank * e:(ps.ep_rank + 1) * e] if full.shape[0] == cfg.num_experts else full
        if tp > 1:
            return full.chunk(tp, dim=1)[tr].contiguous()
    return full


def unshard_tp(name: str, parts: list[torch.Tensor], cfg: ModelConfig) -> torch.Tensor:
    """Inverse of `shard_for_rank` along TP for one parameter (parts ordered by tp rank)."""
    if len(parts) == 1:
        return parts[0]
    last = name.rsplit(".", 1)[-1]
    if last in ("wqkv", "bqkv"):
        from .qwen3 import unshard_qkv
        return unshard_qkv(parts, cfg)
    if last == "wo":
        return torch.cat(parts, dim=1)
    if last == "lm_head":
        return torch.cat(parts, dim=0)
    if last == "w13" and parts[0].dim() == 2:
        gs, us = zip(*[p.chunk(2, dim=0) for p in parts])
        return torch.cat(list(gs) + list(us), 0)
    if last == "w2" and parts[0].dim() == 2:
        return torch.cat(parts, dim=1)
    return parts[0]  # replicated


def load_named_into_model(model, named_tensors: Iterable[tuple[str, torch.Tensor]], cfg: ModelConfig, ps):
    """Copy tensors into a model. Accepts this package's names (shard or full) or HF names (full)."""
    named = list(named_tensors)
    params = dict(model.named_parameters_global() if hasattr(model, "named_parameters_global") else model.named_parameters())
    if named and (named[0][0].startswith("model.") or named[0][0].startswith("lm_head")):
        from ..weight_update.quant_export import dequantize_named, is_quantized_stream

        if is_quantized_stream(named):              # fp8 / mxfp8 / nvfp4 / int4 export formats decode on arrival
            named = dequantize_named(named, next(iter(params.values())).dtype)
        named = list(hf_state_to_ours(dict(named), cfg).items())
    for n, t in named:
        if n not in params:
            continue
        p = params[n]
        if tuple(t.shape) != tuple(p.shape):
            t = shard_for_rank(n, t, cfg, ps)
        assert tuple(t.shape) == tuple(p.shape), f"{n}: got {tuple(t.shape)}, model has {tuple(p.shape)}"
        if type(p.data) is not torch.Tensor:           # an FSDP-sharded parameter takes its slice of the full tensor
            from ..train.fsdp import copy_into

            copy_into(p, t)
        elif t.data_ptr() != p.data.data_ptr():
            p.data.copy_(t)


# ---- Megatron ⇄ ours -------------------------------------------------------------------------

def megatron_qkv_to_ours(w: torch.Tensor, cfg: ModelConfig) -> torch.Tensor:
    """Megatron `linear_qkv.weight` [(g·(r+2))·D, H] grouped per KV head → [q; k; v] stacked."""
    g, D = cfg.num_kv_heads, cfg.head_dim
    r = cfg.num_heads // g
    tail = w.shape[1:]
    x = w.view(g, r + 2, D, *tail)
    q = x[:, :r].reshape(g * r * D, *tail)
    k = x[:, r].reshape(g * D, *tail)
    v = x[:, r + 1].reshape(g * D, *tail)
    return torch.cat([q, k, v], 0)


def ours_qkv_to_megatron(w: torch.Tensor, cfg: ModelConfig) -> torch.Tensor:
    g, D = cfg.num_kv_heads, cfg.head_dim
    r = cfg.num_heads // g
    tail = w.shape[1:]
    q, k, v = w.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
    x = torch.cat([q.view(g, r, D, *tail), k.view(g, 1, D, *tail), v.view(g, 1, D, *tail)], dim=1)
    return x.reshape(g * (r + 2) * D, *tail)


def megatron_name_map(cfg: ModelConfig) -> dict[str, str]:
    """ours → Megatron parameter name (without the `module.module.` wrapper prefix)."""
    m = {"embed": "embedding.word_embeddings.weight", "lm_head": "output_layer.weight",
         "norm": "decoder.final_layernorm.weight"}
    for L in range(cfg.num_layers):
        o, d = f"layers.{L}", f"decoder.layers.{L}"
        m[f"{o}.ln1"] = f"{d}.self_attention.linear_qkv.layer_norm_weight"
        m[f"{o}.attn.wqkv"] = f"{d}.self_attention.linear_qkv.weight"
        m[f"{o}.attn.bqkv"] = f"{d}.self_attention.linear_qkv.bias"
        m[f"{o}.attn.wo"] = f"{d}.self_attention.linear_proj.weight"
        m[f"{o}.attn.q_norm"] = f"{d}.self_attention.q_layernorm.weight"
        m[f"{o}.attn.k_norm"] = f"{d}.self_attention.k_layernorm.weight"
        if cfg.layer_is_moe(L):
            m[f"{o}.ln2"] = f"{d}.pre_mlp_layernorm.weight"
            m[f"{o}.mlp.router"] = f"{d}.mlp.router.weight"
            m[f"{o}.mlp.w13"] = f"{d}.mlp.experts.linear_fc1.weight"   # + expert id suffix
            m[f"{o}.mlp.w2"] = f"{d}.mlp.experts.linear_fc2.weight"
        else:
            m[f"{o}.ln2"] = f"{d}.mlp.linear_fc1.layer_norm_weight"
            m[f"{o}.mlp.w13"] = f"{d}.mlp.linear_fc1.weight"
            m[f"{o}.mlp.w2"] = f"{d}.mlp.linear_fc2.weight"
    return m


def ours_to_megatron(state: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    nm = megatron_name_map(cfg)
    out = {}
    for n, t in state.items():
        if n.endswith("wqkv") or n.endswith("bqkv"):
            out[nm[n]] = ours_qkv_to_megatron(t, cfg)
        elif t.dim() == 3 and (n.endswith("w13") or n.endswith("w2")):
            for e in range(t.shape[0]):
                out[f"{nm[n]}{e}"] = t[e]
        else:
            out[nm[n]] = t
    return out


def megatron_to_ours(state: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    inv = {v: k for k, v in megatron_name_map(cfg).items()}
    out: dict[str, torch.Tensor] = {}
    experts: dict[str, dict[int, torch.Tensor]] = {}
    for n, t in state.items():
        n = re.sub(r"^(module\.)+", "", n)
        m = re.match(r"(.*linear_fc[12]\.weight)(\d+)$", n)
        if m and m.group(1) in inv:
            experts.setdefault(inv[m.group(1)], {})[int(m.group(2))] = t
            continue
        if n not in inv:
            continue
        o = inv[n]
        out[o] = megatron_qkv_to_ours(t, cfg) if o.endswith("wqkv") or o.endswith("bqkv") else t
    for o, d in experts.items():
        out[o] = torch.stack([d[e] for e in sorted(d)])
    return out
