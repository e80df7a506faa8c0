"""Functional op layer.

CUDA tensors run the hand-written sm_100a kernels of the in-tree extension
(`miles_b200.ops.cuda`, built by `miles_b200.ops.build`); CPU tensors run the plain-PyTorch
statements in `reference.py` (the oracle, and the path of the gloo plumbing tests).  There is no
silent fallback: a CUDA tensor with the extension missing raises.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import reference as ref

_cuda = None


def _k():
    """The CUDA op module (autograd wrappers over the extension); imported on first CUDA use."""
    global _cuda
    if _cuda is None:
        from . import cuda as _c  # raises with a build hint when the .so is absent

        _cuda = _c
    return _cuda


def cuda_available() -> bool:
    try:
        _k()
        return torch.cuda.is_available()
    except Exception:
        return False


# ---- dense -----------------------------------------------------------------------------------

def linear(x, w, bias=None):
    if x.is_cuda:
        return _k().linear(x, w, bias)
    return F.linear(x, w, bias)


def linear_fp32(x, w):
    """x·Wᵀ with an fp32 result (LM-head logits for sampling: no bf16 rounding of the logits)."""
    if x.is_cuda:
        return _k().linear_fp32(x, w)
    return F.linear(x, w).float()


def linear_dgrad(gy, w):
    """dX = dY · W for y = x·Wᵀ (W [N,K])."""
    if gy.is_cuda:
        return _k().linear_dgrad(gy, w)
    return gy @ w


def linear_wgrad(gy, x):
    """dW = dYᵀ · X (returned in the dtype of x)."""
    if gy.is_cuda:
        return _k().linear_wgrad(gy, x)
    return gy.t() @ x


def embedding(tokens, w):
    return F.embedding(tokens.long(), w)


def rmsnorm(x, w, eps=1e-6):
    if x.is_cuda:
        return _k().rmsnorm(x, w, eps)
    return ref.rmsnorm(x, w, eps)


def few_token_decode(x, w) -> bool:
    """True when the matrix-vector decode kernels apply to `x · wᵀ`: CUDA bf16, no autograd, a handful of rows."""
    return x.is_cuda and _k().gemv_ok(x, w)


def add_rmsnorm_linear(x, residual, norm_w, eps, w, bias=None, want_normed=False, out_fp32=False):
    """rmsnorm(x + residual) · wᵀ in one kernel (only where `few_token_decode` holds).
    Returns (y, x + residual, normalised activations or None)."""
    y, res, xn = _k().add_rmsnorm_linear(x, residual, norm_w, eps, w, bias, want_normed, out_fp32)
    return y, (x if res is None else res), xn


def add_rmsnorm(x, residual, w, eps=1e-6):
    """(x + residual) → (rmsnorm(sum), sum); residual None means x starts the stream."""
    if residual is None:
        return rmsnorm(x, w, eps), x
    if x.is_cuda:
        return _k().add_rmsnorm(x, residual, w, eps)
    return ref.add_rmsnorm(x, residual, w, eps)


def swiglu(gate_up):
    if gate_up.is_cuda:
        return _k().swiglu(gate_up)
    return ref.swiglu(gate_up)


def qk_norm_rope(q, k, q_w, k_w, positions, theta, eps=1e-6):
    """Per-head RMSNorm of q and k (when weights given) followed by NeoX rotary embedding."""
    if q.is_cuda:
        return _k().qk_norm_rope(q, k, q_w, k_w, positions, theta, eps)
    if q_w is not None:
        q, k = ref.rmsnorm(q, q_w, eps), ref.rmsnorm(k, k_w, eps)
    return ref.rope(q, positions, theta), ref.rope(k, positions, theta)


def qk_norm_rope_cache(q, k, v, q_w, k_w, positions, theta, eps, k_cache, v_cache, slot_mapping):
    """`qk_norm_rope` followed by `kv_cache_write` of (rotated k, v); one kernel on the GPU inference path."""
    if q.is_cuda:
        return _k().qk_norm_rope_cache(q, k, v, q_w, k_w, positions, theta, eps, k_cache, v_cache, slot_mapping)
    q, k = qk_norm_rope(q, k, q_w, k_w, positions, theta, eps)
    kv_cache_write(k, v, k_cache, v_cache, slot_mapping)
    return q, k


def rope(x, positions, theta, inverse=False):
    if x.is_cuda:
        return _k().rope(x, positions, theta, inverse)
    return ref.rope(x, positions, theta, inverse)


# ---- router / MoE ----------------------------------------------------------------------------

def router_topk(logits, k, normalize=True):
    if logits.is_cuda:
        return _k().router_topk(logits, k, normalize)
    return ref.router_topk(logits, k, normalize)


def gather_router_weights(probs, idx, normalize=True):
    return ref.gather_router_weights(probs, idx, normalize)


def moe_ffn(x, w13, w2, topk_w, topk_idx):
    if x.is_cuda:
        return _k().moe_ffn(x, w13, w2, topk_w, topk_idx)
    return ref.moe_ffn(x, w13, w2, topk_w, topk_idx)


# ---- attention -------------------------------------------------------------------------------

def attention_varlen(q, k, v, cu_seqlens, max_seqlen=0, causal=True):
    if q.is_cuda:
        return _k().attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal)
    return ref.attention_varlen(q, k, v, cu_seqlens, causal)


def kv_cache_write(k, v, k_cache, v_cache, slot_mapping):
    """Scatter new K/V rows [T,Hkv,D] into the paged cache [blocks, block_size, Hkv, D]."""
    if k.is_cuda:
        return _k().kv_cache_write(k, v, k_cache, v_cache, slot_mapping)
    kc = k_cache.view(-1, *k_cache.shape[2:])
    vc = v_cache.view(-1, *v_cache.shape[2:])
    kc[slot_mapping.long()] = k.detach().to(kc.dtype)
    vc[slot_mapping.long()] = v.detach().to(vc.dtype)


def paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens=None, max_q_len=1, extend=None):
    if q.is_cuda:
        return _k().paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens, max_q_len, extend)
    return ref.paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens=q_lens)


# ---- loss head -------------------------------------------------------------------------------

def logprob_entropy(hidden, w, targets, temperature=1.0, with_entropy=False):
    """(log p(target), entropy | None) without materialising [T,V] logits on the GPU path."""
    if hidden.is_cuda:
        return _k().logprob_entropy(hidden, w, targets, temperature, with_entropy)
    return ref.logprob_entropy(hidden, w, targets, temperature, with_entropy=with_entropy)


# ---- optimizer / quant -----------------------------------------------------------------------

def adamw_step(master, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale=1.0, param_out=None):
    if master.is_cuda:
        return _k().adamw_step(master, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step,
                               grad_scale, param_out)
    return ref.adamw_step(master, grad, exp_avg, exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                          weight_decay=weight_decay, step=step, grad_scale=grad_scale, param_out=param_out)


def mxfp8_quant(x):
    return _k().mxfp8_quant(x) if x.is_cuda else ref.mxfp8_quant(x)


def fp8_blockwise_quant(w):
    return _k().fp8_blockwise_quant(w) if w.is_cuda else ref.fp8_blockwise_quant(w)


def mxfp8_dequant(q, scales):
    """1×32-block MXFP8 (e4m3 payload, e8m0 scales) → bf16."""
    from . import extra

    return extra.fp8_dequant(q.reshape(-1, q.shape[-1]), scales.reshape(-1, scales.shape[-1])).reshape(q.shape)


def fp8_blockwise_dequant(q, scale_inv):
    """128×128-block FP8 (e4m3 payload, fp32 scale_inv) → bf16."""
    from . import extra

    return extra.fp8_dequant(q, scale_inv)


def int4_fake_quant(x, block_m=1, block_n=32, symmetric=True):
    if x.is_cuda:
        return _k().int4_fake_quant(x, block_m, block_n, symmetric)
    return ref.int4_fake_quant(x, block_m, block_n, symmetric)


def nvfp4_qdq(x, global_amax=None, four_over_six=False):
    return _k().nvfp4_qdq(x, global_amax, four_over_six) if x.is_cuda else ref.nvfp4_qdq(x, global_amax, four_over_six=four_over_six)


class _StraightThrough(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mode):
        if x.is_cuda and x.dtype == torch.bfloat16:
            return _k().C.block_fake_quant(x.contiguous(), {"fp8": 0, "fp4": 1, "compressed_kv": 2}[mode])
        return ref.block_fake_quant(x, mode)

    @staticmethod
    def backward(ctx, g):
        return g, None


def block_fake_quant(x, mode: str = "fp8"):
    """Quantise → dequantise per block along the last axis with a straight-through gradient: `fp8` / `fp4` (1×32 blocks,
    power-of-two scales: MXFP8 / MXFP4 numerics for quantisation-aware training), `compressed_kv` (1×16 blocks, e4m3
    scales, e2m1 payload)."""
    assert mode in ("fp8", "fp4", "compressed_kv")
    return _StraightThrough.apply(x, mode)
