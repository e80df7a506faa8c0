"""Packed low-bit export formats applied to HF-named tensors during weight sync and checkpoint conversion.

* `nvfp4` (ModelOpt layout): `<w>.weight` uint8 [M, K/2] — two e2m1 codes per byte, even column in the low nibble —
  `<w>.weight_scale` float8_e4m3fn [M, K/16] block scales, `<w>.weight_scale_2` fp32 scalar per tensor
  (amax / (448·6)); a gate/up pair (`gate_proj`/`up_proj`, `w1`/`w3`) shares one scalar because serving engines fuse
  the two matrices.  Eligible: routed-expert projections of decoder layers, minus the ignore rules (literal module
  prefixes or `re:` patterns) and minus a bf16 head / tail of layers
  (reference: miles/backends/megatron_utils/megatron_to_hf/processors/quantizer_nvfp4.py:16-204).
  `four_over_six`: per block, quantise once with the block maximum mapped to 6 and once mapped to 4 (finer steps for
  blocks whose values crowd the upper half) and keep the candidate with the smaller squared error
  (reference: miles/kernels/quant/nvfp4_qdq.py:41-73).
* `int4` (compressed-tensors pack-quantized): group-wise integer codes in [-8, 7] (symmetric) or [0, 15] with a zero
  point, eight codes per int32 along K in ascending nibble order: `<w>.weight_packed` int32 [M, K/8],
  `<w>.weight_scale` [M, K/g], `<w>.weight_shape` int64 [2] (+ `<w>.weight_zero_point` int32 packed along M when asymmetric)
  (reference: processors/quantizer_compressed_tensors.py:150-303).

Both come with their inverse so that a test — and a consumer without the serving kernels — can check that what was
exported decodes to exactly what fake-quantised training saw (`ops.nvfp4_qdq`, `ops.int4_fake_quant`).
"""
from __future__ import annotations

import re

import torch

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
FP8_MAX, FP4_MAX = 448.0, 6.0
GATED = {".gate_proj.weight": "gate", ".up_proj.weight": "up", ".w1.weight": "gate", ".w3.weight": "up"}


# ---- NVFP4 -----------------------------------------------------------------------------------------------------------

def e2m1_codes(a: torch.Tensor) -> torch.Tensor:
    """|value| ≤ 6 → code 0..7, round to nearest, ties to the even code (as `cvt.rn.satfinite.e2m1x2`)."""
    a = a.clamp(max=FP4_MAX)
    return ((a > 0.25).to(torch.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5) + (a > 5.0)).to(torch.uint8)


def _nvfp4_blocks(xf: torch.Tensor, gscale: torch.Tensor, target: float):
    """One candidate: block max → `target` (6 or 4).  Returns (codes uint8 [N,16], e4m3 block scale [N,1], dequantised)."""
    amax = xf.abs().amax(-1, keepdim=True)
    sb = (amax / target * gscale).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    dec = sb.float() / gscale
    scaled = xf * torch.where(dec > 0, 1.0 / dec, torch.zeros_like(dec))       # multiply by the reciprocal, as the kernel does
    codes = e2m1_codes(scaled.abs())
    deq = E2M1.to(xf.device)[codes.long()] * scaled.sign() * dec
    return codes | ((scaled < 0).to(torch.uint8) << 3), sb, deq


def nvfp4_quantize(w: torch.Tensor, global_amax: torch.Tensor | None = None, four_over_six: bool = False):
    """[M, K] → (packed uint8 [M, K/2], block scales e4m3 [M, K/16], fp32 scalar `weight_scale_2`)."""
    M, K = w.shape
    assert K % 16 == 0, f"NVFP4 needs the last dimension divisible by 16, got {K}"
    xf = w.float().reshape(-1, 16)
    gamax = (w.float().abs().max() if global_amax is None else global_amax.float()).clamp_min(1e-12)
    gscale = (FP8_MAX * FP4_MAX) / gamax
    codes, sb, deq = _nvfp4_blocks(xf, gscale, FP4_MAX)
    if four_over_six:
        c4, s4, d4 = _nvfp4_blocks(xf, gscale, 4.0)
        better = ((d4 - xf) ** 2).sum(-1, keepdim=True) < ((deq - xf) ** 2).sum(-1, keepdim=True)
        codes, sb = torch.where(better, c4, codes), torch.where(better, s4.float(), sb.float()).to(torch.float8_e4m3fn)
    codes = codes.reshape(M, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, sb.reshape(M, K // 16), (1.0 / gscale).to(torch.float32)


def nvfp4_dequantize(packed: torch.Tensor, block_scale: torch.Tensor, scale_2: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    M, half = packed.shape
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(M, half * 2)
    mag = E2M1.to(packed.device)[(codes & 7).long()]
    val = torch.where((codes & 8) > 0, -mag, mag)
    dec = (block_scale.float() * scale_2.float()).repeat_interleave(16, dim=1)
    return (val * dec).to(dtype)


def is_ignored(name: str, rules: list[str]) -> bool:
    """`name` (a module or tensor name) matches a literal rule when it equals it or lies below it; `re:` rules are regexes."""
    mod = name[: -len(".weight")] if name.endswith(".weight") else name
    for r in rules or []:
        if r.startswith("re:"):
            if re.match(r[3:], name) or re.match(r[3:], mod):
                return True
        elif mod == r or mod.startswith(r + ".") or name == r:
            return True
    return False


_EXPERT = re.compile(r"model\.layers\.(\d+)\.mlp\.experts\.\d+\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")


def nvfp4_eligible(name: str, t: torch.Tensor, *, ignore: list[str] | None = None, num_layers: int | None = None,
                   bf16_head: int = 0, bf16_tail: int = 0, all_linears: bool = False) -> bool:
    if t.dim() != 2 or not name.endswith(".weight") or t.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        return False
    m = _EXPERT.match(name)
    if m is None and not all_linears:
        return False
    if m is None and (not re.match(r"model\.layers\.(\d+)\.", name) or "norm" in name or name.endswith("mlp.gate.weight")):
        return False
    layer = int(re.match(r"model\.layers\.(\d+)\.", name).group(1))
    if num_layers is not None and (layer < bf16_head or layer >= num_layers - bf16_tail):
        return False
    if is_ignored(name, ignore or []):
        return False
    if t.shape[-1] % 16:
        raise ValueError(f"NVFP4 needs the last dimension divisible by 16 ({name}: {tuple(t.shape)})")
    return True


def export_nvfp4(named: list[tuple[str, torch.Tensor]], **rules) -> list[tuple[str, torch.Tensor]]:
    four_over_six = rules.pop("four_over_six", False)
    pair_strict = rules.pop("pair_strict", True)
    pairs: dict[str, dict[str, torch.Tensor]] = {}
    for n, t in named:
        for sfx, role in GATED.items():
            if n.endswith(sfx) and nvfp4_eligible(n, t, **rules):
                pairs.setdefault(n[: -len(sfx)], {})[role] = t
    shared = {}
    for base, roles in pairs.items():
        if set(roles) != {"gate", "up"}:
            if not pair_strict:               # a shard-by-shard conversion may see one half only: it keeps its own scale
                continue
            raise ValueError(f"NVFP4 quantises gate and up together (one shared tensor scale); only {sorted(roles)} of {base} in this batch")
        shared[base] = torch.maximum(roles["gate"].float().abs().max(), roles["up"].float().abs().max())
    out = []
    for n, t in named:
        if not nvfp4_eligible(n, t, **rules):
            out.append((n, t))
            continue
        base = next((n[: -len(s)] for s in GATED if n.endswith(s)), None)
        q, sb, s2 = nvfp4_quantize(t, shared.get(base), four_over_six)
        out += [(n, q), (n[: -len(".weight")] + ".weight_scale", sb), (n[: -len(".weight")] + ".weight_scale_2", s2)]
    return out


# ---- compressed-tensors int4 --------------------------------------------------------------------------------------

def pack_int32(codes: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """Unsigned codes [R, C] → int32 [R, ceil(C / (32/bits))], code j of a word in bits [j·bits, (j+1)·bits)."""
    per = 32 // bits
    R, C = codes.shape
    pad = (-C) % per
    if pad:
        codes = torch.nn.functional.pad(codes, (0, pad))
    c = codes.reshape(R, -1, per).to(torch.int64)
    shifts = torch.arange(per, device=codes.device, dtype=torch.int64) * bits
    word = (c << shifts).sum(-1)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def unpack_int32(packed: torch.Tensor, cols: int, bits: int = 4) -> torch.Tensor:
    per = 32 // bits
    w = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, device=packed.device, dtype=torch.int64) * bits
    c = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return c.reshape(packed.shape[0], -1)[:, :cols]


def int4_quantize(w: torch.Tensor, group_size: int = 32, symmetric: bool = True):
    M, K = w.shape
    assert K % group_size == 0, f"group size {group_size} must divide K = {K}"
    x = w.float().reshape(M, K // group_size, group_size)
    if symmetric:
        scale = (x.abs().amax(-1, keepdim=True) / 7.0).clamp_min(1e-8)
        q = torch.round(x / scale).clamp(-8, 7)
        codes, zp = (q + 8).to(torch.uint8), None
    else:
        lo, hi = x.amin(-1, keepdim=True), x.amax(-1, keepdim=True)
        scale = ((hi - lo) / 15.0).clamp_min(1e-8)
        zp = torch.round(-lo / scale).clamp(0, 15)
        codes = torch.round(x / scale + zp).clamp(0, 15).to(torch.uint8)
    out = {"weight_packed": pack_int32(codes.reshape(M, K)), "weight_scale": scale.reshape(M, -1).to(w.dtype),
           "weight_shape": torch.tensor([M, K], dtype=torch.int64)}
    if zp is not None:
        out["weight_zero_point"] = pack_int32(zp.reshape(M, -1).t().contiguous().to(torch.uint8)).t().contiguous()
    return out


def int4_dequantize(parts: dict, dtype=torch.bfloat16) -> torch.Tensor:
    M, K = (int(v) for v in parts["weight_shape"])
    codes = unpack_int32(parts["weight_packed"], K).float()
    scale = parts["weight_scale"].float()
    g = K // scale.shape[1]
    if "weight_zero_point" in parts:
        zp = unpack_int32(parts["weight_zero_point"].t().contiguous(), M).t().float()
        val = (codes.reshape(M, -1, g) - zp.unsqueeze(-1)) * scale.unsqueeze(-1)
    else:
        val = (codes.reshape(M, -1, g) - 8.0) * scale.unsqueeze(-1)
    return val.reshape(M, K).to(dtype)


def int4_eligible(name: str, t: torch.Tensor, ignore: list[str] | None = None, targets: list[str] | None = None) -> bool:
    if t.dim() != 2 or not name.endswith(".weight") or any(s in name for s in ("embed_tokens", "lm_head", "norm", "mlp.gate.weight")):
        return False
    if targets and not any(re.search(p, name) for p in targets):
        return False
    return not is_ignored(name, ignore or [])


def export_int4(named, group_size: int = 32, symmetric: bool = True, ignore=None, targets=None):
    out = []
    for n, t in named:
        if not int4_eligible(n, t, ignore, targets) or t.shape[1] % group_size:
            out.append((n, t))
            continue
        base = n[: -len(".weight")]
        out += [(f"{base}.{k}", v) for k, v in int4_quantize(t, group_size, symmetric).items()]
    return out


def quant_config(mode: str, *, group_size: int = 32, symmetric: bool = True, ignore=None, four_over_six: bool = False) -> dict:
    if mode == "nvfp4":
        return {"quantization_config": {"quant_method": "modelopt", "quant_algo": "NVFP4", "group_size": 16,
                                        "kv_cache_quant_algo": None, "ignore": list(ignore or []),
                                        **({"block_scale_rule": "four_over_six"} if four_over_six else {})}}
    if mode == "int4":
        return {"quantization_config": {
            "quant_method": "compressed-tensors", "format": "pack-quantized", "ignore": list(ignore or ["lm_head"]),
            "config_groups": {"group_0": {"targets": ["Linear"], "weights": {
                "num_bits": 4, "type": "int", "symmetric": symmetric, "strategy": "group", "group_size": group_size}}}}}
    return {}


# ---- the receiving side ---------------------------------------------------------------------------------------------

def dequantize_named(named, dtype=torch.bfloat16) -> list[tuple[str, torch.Tensor]]:
    """HF-named tensors in any of the export formats → plain `<w>.weight` tensors holding the quantised values.  This
    engine computes in bf16, so a quantised stream is served by decoding it on arrival: the values the policy samples with
    are exactly those a low-precision serving kernel would multiply with."""
    from .. import ops

    named = list(named)
    d = dict(named)
    companions = (".weight_scale", ".weight_scale_2", ".weight_scale_inv", ".weight_shape", ".weight_zero_point", ".input_scale")
    out = []
    for n, t in named:
        if n.endswith(companions):
            continue
        if n.endswith(".weight_packed"):
            base = n[: -len(".weight_packed")]
            parts = {k: d[f"{base}.{k}"] for k in ("weight_packed", "weight_scale", "weight_shape", "weight_zero_point") if f"{base}.{k}" in d}
            out.append((base + ".weight", int4_dequantize(parts, dtype)))
        elif n.endswith(".weight") and t.dtype == torch.uint8 and n[: -len(".weight")] + ".weight_scale_2" in d:
            base = n[: -len(".weight")]
            out.append((n, nvfp4_dequantize(t, d[base + ".weight_scale"], d[base + ".weight_scale_2"], dtype)))
        elif n + "_scale_inv" in d:
            s = d[n + "_scale_inv"]
            val = ops.mxfp8_dequant(t, s).reshape(t.shape) if s.dtype == torch.uint8 else ops.fp8_blockwise_dequant(t, s)
            out.append((n, val.to(dtype)))
        else:
            out.append((n, t))
    return out


def is_quantized_stream(named) -> bool:
    return any(n.endswith((".weight_packed", ".weight_scale_2", ".weight_scale_inv")) for n, _ in named)
