"""HF checkpoint names of the model families in `families.py` (the role of the reference's per-architecture weight
bridges, miles_plugins/mbridge/{deepseek_v32,glm4moe,qwen3_next,kimi_k3,…}.py).

`to_hf` / `from_hf` extend the Qwen3 converter (`convert.py`): the tensors the Qwen3 layout already knows (embeddings,
norms, fused QKV, gate/up stacks, routed experts, router) go through it; the family-specific tensors are renamed, and
split or fused where HF stores them differently:

    attn.wq_a / q_a_norm / wq_b / wq      self_attn.q_a_proj / q_a_layernorm / q_b_proj / q_proj
    attn.wkv_a / kv_a_norm / wkv_b        self_attn.kv_a_proj_with_mqa / kv_a_layernorm / kv_b_proj
    attn.wq_idx / wk_idx / k_idx_norm / w_idx   self_attn.indexer.wq_b / wk / k_norm / weights_proj
    attn.w_gate                           fused into self_attn.q_proj as [heads, 2·head_dim, hidden] (query | gate per head)
    attn.w_qkvz / w_ba / conv / A_log / dt_bias / o_norm / wo (linear attention)
                                          linear_attn.in_proj_qkvz / in_proj_ba / conv1d ([C, 1, K]) / A_log / dt_bias / norm / out_proj
    mlp.e_bias                            mlp.gate.e_score_correction_bias
    mlp.shared.w13 / w2                   mlp.shared_experts.gate_proj + up_proj / down_proj
    hc.<block>_<pre|post|res>             hyper_connection.<block>.<pre|post|res>   (no HF counterpart: kept under this name)
"""
from __future__ import annotations

import re

import torch

from . import convert as base
from .families import FamilyConfig

_ATTN_RENAME = {
    "wq_a": "q_a_proj.weight", "q_a_norm": "q_a_layernorm.weight", "wq_b": "q_b_proj.weight", "wq": "q_proj.weight",
    "wkv_a": "kv_a_proj_with_mqa.weight", "kv_a_norm": "kv_a_layernorm.weight", "wkv_b": "kv_b_proj.weight",
    "wq_idx": "indexer.wq_b.weight", "wk_idx": "indexer.wk.weight", "k_idx_norm": "indexer.k_norm.weight",
    "w_idx": "indexer.weights_proj.weight",
}
_LINEAR_RENAME = {
    "w_qkvz": "in_proj_qkvz.weight", "w_ba": "in_proj_ba.weight", "A_log": "A_log", "dt_bias": "dt_bias",
    "o_norm": "norm.weight", "wo": "out_proj.weight",
}


def _kind(cfg: FamilyConfig, layer: int) -> str:
    return cfg.layer_type(layer) if isinstance(cfg, FamilyConfig) else "full"


def to_hf(name: str, tensor: torch.Tensor, cfg, *, expert_offset: int = 0, gate: torch.Tensor | None = None):
    """One full tensor of this package's layout → [(hf_name, tensor)].  For a gated full-attention layer pass the layer's
    `attn.w_gate` as `gate` together with `attn.wqkv` (HF fuses the gate into q_proj); `attn.w_gate` on its own is sent as
    `self_attn.gate_proj.weight`, which `from_hf` also accepts."""
    m = re.match(r"layers\.(\d+)\.(.+)", name)
    if not m:
        return base.to_hf(name, tensor, cfg, expert_offset=expert_offset, _plain=True)
    L, rest = int(m.group(1)), m.group(2)
    pre, kind = f"model.layers.{L}", _kind(cfg, L)
    if rest.startswith("hc."):
        block, w = rest[3:].rsplit("_", 1)
        return [(f"{pre}.hyper_connection.{block}.{w}", tensor)]
    if rest == "mlp.e_bias":
        return [(f"{pre}.mlp.gate.e_score_correction_bias", tensor)]
    if rest == "mlp.shared.w13":
        g, u = tensor.chunk(2, 0)
        return [(f"{pre}.mlp.shared_experts.gate_proj.weight", g), (f"{pre}.mlp.shared_experts.up_proj.weight", u)]
    if rest == "mlp.shared.w2":
        return [(f"{pre}.mlp.shared_experts.down_proj.weight", tensor)]
    if rest.startswith("attn."):
        p = rest[5:]
        if kind in ("gdn", "kda"):
            if p == "conv":
                return [(f"{pre}.linear_attn.conv1d.weight", tensor.unsqueeze(1))]
            return [(f"{pre}.linear_attn.{_LINEAR_RENAME[p]}", tensor)]
        if kind in ("mla", "dsa") and p in _ATTN_RENAME:
            return [(f"{pre}.self_attn.{_ATTN_RENAME[p]}", tensor)]
        if p == "w_gate":
            # tensor-at-a-time callers (weight sync) send the gate under its own name; `state_to_hf` fuses it into q_proj
            return [(f"{pre}.self_attn.gate_proj.weight", tensor)]
        if p == "wqkv" and gate is not None:
            q, k, v = tensor.split([cfg.q_size, cfg.kv_size, cfg.kv_size], 0)
            d, H = cfg.head_dim, cfg.hidden_size
            fused = torch.cat([q.view(cfg.num_heads, d, H), gate.view(cfg.num_heads, d, H)], 1).reshape(2 * cfg.q_size, H)
            return [(f"{pre}.self_attn.q_proj.weight", fused), (f"{pre}.self_attn.k_proj.weight", k),
                    (f"{pre}.self_attn.v_proj.weight", v)]
    return base.to_hf(name, tensor, cfg, expert_offset=expert_offset, _plain=True)


def state_to_hf(state: dict[str, torch.Tensor], cfg) -> dict[str, torch.Tensor]:
    """Whole (un-sharded) state dict of a family model → HF names."""
    out = {}
    for name, t in state.items():
        gate = None
        if name.endswith("attn.wqkv"):
            gate = state.get(name[:-4] + "w_gate")
        if name.endswith("attn.w_gate") and (name[:-6] + "wqkv") in state:
            continue
        for hn, ht in to_hf(name, t, cfg, gate=gate):
            out[hn] = ht
    return out


def from_hf(hf: dict[str, torch.Tensor], cfg) -> dict[str, torch.Tensor]:
    """HF tensors → this package's names (inverse of `state_to_hf`)."""
    hf = dict(hf)
    ours: dict[str, torch.Tensor] = {}
    inv_attn = {v: k for k, v in _ATTN_RENAME.items()}
    inv_lin = {v: k for k, v in _LINEAR_RENAME.items()}
    for hn in list(hf):
        m = re.match(r"model\.layers\.(\d+)\.(.+)", hn)
        if not m or hn not in hf:
            continue
        L, rest = int(m.group(1)), m.group(2)
        kind, pre = _kind(cfg, L), f"layers.{L}"
        t = hf[hn]
        if rest.startswith("hyper_connection."):
            block, w = rest[len("hyper_connection."):].split(".")
            ours[f"{pre}.hc.{block}_{w}"] = hf.pop(hn)
        elif rest == "self_attn.gate_proj.weight":
            ours[f"{pre}.attn.w_gate"] = hf.pop(hn)
        elif rest == "mlp.gate.e_score_correction_bias":
            ours[f"{pre}.mlp.e_bias"] = hf.pop(hn)
        elif rest == "mlp.shared_experts.gate_proj.weight":
            up = hf.pop(f"model.layers.{L}.mlp.shared_experts.up_proj.weight")
            ours[f"{pre}.mlp.shared.w13"] = torch.cat([hf.pop(hn), up], 0)
        elif rest == "mlp.shared_experts.down_proj.weight":
            ours[f"{pre}.mlp.shared.w2"] = hf.pop(hn)
        elif rest.startswith("linear_attn."):
            p = rest[len("linear_attn."):]
            ours[f"{pre}.attn.conv" if p == "conv1d.weight" else f"{pre}.attn.{inv_lin[p]}"] = (
                hf.pop(hn).squeeze(1) if p == "conv1d.weight" else hf.pop(hn))
        elif rest.startswith("self_attn.") and kind in ("mla", "dsa") and rest[len("self_attn."):] in inv_attn:
            ours[f"{pre}.attn.{inv_attn[rest[len('self_attn.'):]]}"] = hf.pop(hn)
        elif (rest == "self_attn.q_proj.weight" and kind == "full" and getattr(cfg, "attn_output_gate", False)
              and t.shape[0] == 2 * cfg.q_size):
            d, H = cfg.head_dim, cfg.hidden_size
            qg = hf.pop(hn).view(cfg.num_heads, 2 * d, H)
            hf[hn] = qg[:, :d].reshape(cfg.q_size, H)
            ours[f"{pre}.attn.w_gate"] = qg[:, d:].reshape(cfg.q_size, H)
    hf = {k: v for k, v in hf.items() if "up_proj" not in k or "shared_experts" not in k}
    ours.update(base.hf_state_to_ours(hf, cfg, _plain=True))
    return ours


def full_state(model) -> dict[str, torch.Tensor]:
    """Model-wide named tensors of a single-rank family model (parameters, plus the non-trainable selection bias)."""
    return {n: p.detach() for n, p in model.named_parameters_global()}
