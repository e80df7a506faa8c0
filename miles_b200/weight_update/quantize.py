"""Weight quantisers applied during export / weight sync.

* `fp8`:  128×128-block e4m3 with fp32 `weight_scale_inv` (reference: processors/quantizer_fp8.py:16-177,
  kernel miles/kernels/quant/fp8_blockwise.py:24-79).
* `mxfp8`: 1×32-block e4m3 with uint8 e8m0 `weight_scale_inv`
  (reference: processors/quantizer_mxfp8.py:6-114, miles/utils/mxfp8.py:48-78).
* `nvfp4`, `int4`: packed export formats, see `quant_export.py`.
Only 2-D projection weights are quantised; embeddings, norms, the router gate and the LM head stay in
bf16 (the reference's skip list, miles/utils/mxfp8.py:7-20).
"""
from __future__ import annotations

import torch

from .. import ops

SKIP_SUBSTRINGS = ("embed_tokens", "lm_head", "norm", "mlp.gate.weight", "bias", "router")


def should_quantize(name: str, t: torch.Tensor) -> bool:
    if t.dim() != 2 or not name.endswith(".weight"):
        return False
    return not any(s in name for s in SKIP_SUBSTRINGS)


def quantize_hf_tensors(named: list[tuple[str, torch.Tensor]], mode: str, **options) -> list[tuple[str, torch.Tensor]]:
    if mode in ("nvfp4", "int4"):                    # packed export formats with their own eligibility rules
        from . import quant_export

        return (quant_export.export_nvfp4 if mode == "nvfp4" else quant_export.export_int4)(list(named), **options)
    out: list[tuple[str, torch.Tensor]] = []
    for n, t in named:
        if not should_quantize(n, t):
            out.append((n, t))
            continue
        if mode == "fp8":
            q, s = ops.fp8_blockwise_quant(t)
        elif mode == "mxfp8":
            if t.shape[1] % 32:            # 1×32 blocks must not straddle rows: such a tensor stays in bf16
                out.append((n, t))
                continue
            q, s = ops.mxfp8_quant(t)
        else:
            raise ValueError(f"unknown quantisation {mode}")
        out.append((n, q))
        out.append((n + "_scale_inv", s))
    return out


def hf_quant_config(mode: str) -> dict:
    if mode == "fp8":
        return {"quantization_config": {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic",
                                        "weight_block_size": [128, 128]}}
    if mode == "mxfp8":
        return {"quantization_config": {"quant_method": "mxfp8", "fmt": "e4m3", "weight_block_size": [1, 32],
                                        "scale_fmt": "ue8m0"}}
    if mode in ("nvfp4", "int4"):
        from . import quant_export

        return quant_export.quant_config(mode)
    return {}
