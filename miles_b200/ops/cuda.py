"""CUDA execution of the op layer: autograd Functions over the sm_100a extension (`miles_b200_C`).

Importing this module loads the in-tree `.so`; it raises if the extension has not been built, so a
GPU run can never silently fall back to library kernels.  All tensors are bf16 unless noted; fp32 is
used for statistics, router maths, gradients-in-accumulation and optimizer state.
"""
from __future__ import annotations

import math
import os

import torch

from . import build as _build
from . import reference as ref

C = _build.load()

# the debug build of the extension (MILES_DEBUG_KERNELS=1, csrc/debug.cuh): kernels check the indices they take from tensors
# against limits published here, record violations and skip the access
DEBUG_KERNELS = bool(C.is_debug_build()) if hasattr(C, "is_debug_build") else False
_published: dict[int, int] = {}
LIMIT_KV_SLOTS, LIMIT_MOE_PAIRS, LIMIT_KV_BLOCKS = 0, 1, 2


def publish_limit(which: int, value: int) -> None:
    if DEBUG_KERNELS and _published.get(which) != int(value):
        C.bounds_set_limit(int(which), int(value))
        _published[which] = int(value)


def bounds_report(clear: bool = True) -> list[dict]:
    """Index violations seen by the debug build since the last clearing report: one entry per translation unit that saw any."""
    if not DEBUG_KERNELS:
        return []
    unit = {0: "elementwise.cu", 1: "moe.cu", 2: "paged_decode.cu"}
    return [{"unit": unit[int(r[0])], "count": int(r[1]), "code": int(r[2]), "index": int(r[3]), "limit": int(r[4])}
            for r in C.bounds_report(bool(clear)) if r[1] > 0]

BF16 = torch.bfloat16


def check_error_flag(like: torch.Tensor | None = None) -> int:
    """Value of the device error flag raised by a kernel whose bounded wait expired (0 = healthy).
    Synchronises the device; call at step boundaries and in tests, not per op."""
    t = like if like is not None else torch.empty(0, device="cuda")
    return int(C.error_flag(t).item())


def launch_count() -> int:
    """Number of kernel-launcher calls made by this extension so far (CUDA-graph replays add their captured count)."""
    return int(C.launch_count())


def _c(x: torch.Tensor) -> torch.Tensor:
    return x if x.is_contiguous() else x.contiguous()


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------

def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, bias=None, out_dtype=None,
            accumulate: bool = False, force_bn: int = 0) -> torch.Tensor:
    """a [M,K] · b [N,K]ᵀ → [M,N]."""
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and a.dtype == BF16 and b.dtype == BF16 and K % 8 == 0, (a.shape, b.shape, a.dtype)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or BF16, device=a.device)
    if M and N:
        plain = not accumulate and not force_bn
        if plain and M <= GEMV_M and _gemv_k_ok(M, K) and N <= GEMV_MAX_N:
            C.gemv(a, None, None, 0.0, b, bias, out, None, None, bool(b.is_leaf and b.requires_grad))
            return out
        # measured: the operand-swapped kernel wins where its tiles fill the GPU without split-K (wide outputs such as the
        # LM head); with split-K its reduction costs more than the padding rows of the general kernel
        if plain and M <= SMALL_M and K >= 256 and (SMALL_SPLIT or _small_split(M, N, K, small_bt(M)) == 1):
            return _gemm_small(a, b, out, bias, M, N, K)
        split = _pick_split_k(M, N, K) if not force_bn and SPLIT_K else 1
        if split > 1:
            ws, counters = _splitk_workspace(a.device)
            C.gemm_splitk(a, b, out, M, N, K, out.stride(0), accumulate, bias, split, ws, counters)
        else:
            C.gemm(a, b, out, M, N, K, K, K, out.stride(0), False, False, accumulate, bias, force_bn)
    return out


# Decode-sized GEMMs (a handful of 128×64 output tiles over a long K) leave most SMs idle; split-K gives every tile
# several CTAs, each streaming a slice of the weights.  Workspace: fp32 [split, M, N] planes + arrival counters (zero
# between calls; the kernel restores that), one per device, so such GEMMs must not overlap on two streams of one device.
SPLIT_K = os.environ.get("MILES_SPLIT_K", "1") != "0"
_SPLITK_MAX_M, _SPLITK_MAX_TILES = int(os.environ.get("MILES_SPLIT_K_MAX_M", "32")), 74   # measured: wins below ~32 rows
_splitk_ws: dict = {}


def _pick_split_k(M: int, N: int, K: int) -> int:
    if M > _SPLITK_MAX_M or K < 1024:
        return 1
    tiles = ((M + 127) // 128) * ((N + 63) // 64)
    if tiles > _SPLITK_MAX_TILES:
        return 1
    return max(1, min(148 // tiles, K // 512, 16))


def _splitk_workspace(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _splitk_ws:
        # split · M · N ≤ (148 CTAs) · (128 × 64 tile) floats
        _splitk_ws[key] = (torch.empty(148 * 128 * 64, dtype=torch.float32, device=device),
                           torch.zeros(4 * _SPLITK_MAX_TILES * 2, dtype=torch.int32, device=device))
    return _splitk_ws[key]


# A handful of tokens (decode with a nearly drained batch): matrix-vector kernels without pipeline set-up (gemv.cu).
# Up to 16 rows are supported; 0 turns the path off.
GEMV_M = min(16, int(os.environ.get("MILES_GEMV_M", "16")))
GEMV_MAX_N = int(os.environ.get("MILES_GEMV_MAX_N", "32768"))


def _gemv_k_ok(rows: int, K: int) -> bool:
    """The kernel stages the activation rows in shared memory: 8 (or 16) rows of K bf16 next to a 32 KB weight ring."""
    return K % 32 == 0 and (8 if rows <= 8 else 16) * (2 * K + 64) + 32768 <= 200 * 1024


def add_rmsnorm_linear(x, residual, norm_w, eps, w, bias=None, want_normed: bool = False, out_fp32: bool = False):
    """Inference only, ≤ GEMV_M rows: y = rmsnorm(x + residual) · wᵀ in one kernel.
    Returns (y, x + residual or None, normalised activations or None)."""
    K = x.shape[-1]
    x2 = _c(x.reshape(-1, K))
    r2 = _c(residual.reshape(-1, K)) if residual is not None else None
    M, N = x2.shape[0], w.shape[0]
    y = torch.empty(M, N, dtype=torch.float32 if out_fp32 else BF16, device=x.device)
    res_out = torch.empty_like(x2) if r2 is not None else None
    xn = torch.empty_like(x2) if want_normed else None
    C.gemv(x2, r2, norm_w, float(eps), w, bias, y, res_out, xn, bool(w.is_leaf and w.requires_grad))
    shp = x.shape[:-1]
    return (y.view(*shp, N), res_out.view(x.shape) if res_out is not None else None, xn.view(x.shape) if xn is not None else None)


def gemv_ok(x, w) -> bool:
    """True when `add_rmsnorm_linear` applies: bf16, no autograd, few rows, K a multiple of 32."""
    K = x.shape[-1]
    return (GEMV_M > 0 and x.dtype == BF16 and w.dtype == BF16 and not torch.is_grad_enabled() and _gemv_k_ok(x.numel() // K, K)
            and 0 < x.numel() // K <= GEMV_M and w.is_contiguous())


# Decode-sized token counts: the weight rows go on the 128-row side of the MMA and the tokens on the N side in tiles of
# 16/32/64 (gemm_small.cu), so no pipeline byte is spent on padding rows; split-K fills the SMs.  0 turns the path off.
SMALL_M = int(os.environ.get("MILES_SMALL_M", "64"))
SMALL_SPLIT = os.environ.get("MILES_SMALL_SPLIT", "0") == "1"     # also use it where it needs split-K
_SMALL_WS_FLOATS, _SMALL_MAX_TILES = 4 << 20, 4096
_small_ws: dict = {}


def small_bt(rows: int) -> int:
    return 16 if rows <= 16 else 32 if rows <= 32 else 64


def _small_split(M: int, N: int, K: int, bt: int) -> int:
    out_tiles = ((N + 127) // 128) * ((M + bt - 1) // bt)
    kblocks = (K + 63) // 64
    split = max(1, min(round(148 / out_tiles), kblocks // 2, 32))
    if split > 1 and (out_tiles > _SMALL_MAX_TILES or split * M * N > _SMALL_WS_FLOATS):
        return 1
    per = -(-kblocks // split)
    return -(-kblocks // per)          # every slice gets at least one K block


def _gemm_small(a, b, out, bias, M, N, K):
    bt = small_bt(M)
    split = _small_split(M, N, K, bt)
    ws = counters = None
    if split > 1:
        key = a.device.index if a.device.index is not None else torch.cuda.current_device()
        if key not in _small_ws:
            _small_ws[key] = (torch.empty(_SMALL_WS_FLOATS, dtype=torch.float32, device=a.device),
                              torch.zeros(4 * _SMALL_MAX_TILES, dtype=torch.int32, device=a.device))
        ws, counters = _small_ws[key]
    C.gemm_small(a, b, out, M, N, K, out.stride(0), bias, bt, split, ws, counters)
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=None, force_bn: int = 0):
    """a [M,K] · b [K,N] → [M,N] (b read as an MN-major operand; no transpose copy)."""
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[1]
    assert b.shape[0] == K and K % 8 == 0 and N % 8 == 0
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or BF16, device=a.device)
    if M and N:
        C.gemm(a, b, out, M, N, K, K, N, out.stride(0), False, True, False, None, force_bn)
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=None, accumulate=False,
            force_bn: int = 0):
    """a [K,M]ᵀ · b [K,N] → [M,N] (both MN-major: the weight-gradient form, reduction over rows)."""
    a, b = _c(a), _c(b)
    K, M = a.shape
    N = b.shape[1]
    assert b.shape[0] == K and M % 8 == 0 and N % 8 == 0
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or BF16, device=a.device)
    if M and N:
        if K == 0:
            if not accumulate:
                out.zero_()
        else:
            C.gemm(a, b, out, M, N, K, M, N, out.stride(0), True, True, accumulate, None, force_bn)
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shp = shp
        y = gemm_nt(x2, w, bias=bias)
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        gy2 = _c(gy.reshape(-1, gy.shape[-1]))
        gx = gemm_nn(gy2, w).view(ctx.shp) if ctx.needs_input_grad[0] else None
        gw = gemm_tn(gy2, x2) if ctx.needs_input_grad[1] else None
        gb = gy2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return gx, gw, gb


class _LinearMXFP8(torch.autograd.Function):
    """y = MXFP8(x)·MXFP8(W)ᵀ on the block-scaled tensor-core path; gradients use the bf16 GEMMs on the unquantised
    operands (straight-through), the `--fp8-recipe mxfp8` forward of the reference's TE recipe."""

    @staticmethod
    def forward(ctx, x, w, bias):
        from . import extra

        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.save_for_backward(x2, w)
        ctx.has_bias, ctx.shp = bias is not None, shp
        xq, xs = mxfp8_quant(x2)                   # noqa: F821  (defined in cuda_more, imported at the end of this module)
        wq, ws = mxfp8_quant(w)                    # noqa: F821
        y = extra.gemm_mxfp8(xq, xs, wq, ws)
        if bias is not None:
            y = y + bias
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        if not MXFP8_BACKWARD:
            return _Linear.backward(ctx, gy)
        # both gradient GEMMs block-scaled as well: the contraction runs over N (dgrad) and over the tokens (wgrad), so each
        # operand is quantised along THAT axis — the transposed copies are made here, quantised 1×32 along their rows, and the
        # same NT kernel serves all three products (the reference's recipe quantises the transposes the same way,
        # miles/utils/mxfp8.py:48-78)
        from . import extra

        x2, w = ctx.saved_tensors
        gy2 = _c(gy.reshape(-1, gy.shape[-1]))
        M, N = gy2.shape
        K = w.shape[1]
        if N % 128 or M % 128 or K % 128:
            return _Linear.backward(ctx, gy)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gq, gs = mxfp8_quant(gy2)                                  # noqa: F821
            wtq, wts = mxfp8_quant(w.t().contiguous())                 # noqa: F821   [K, N], blocks along N
            gx = extra.gemm_mxfp8(gq, gs, wtq, wts).view(ctx.shp)
        if ctx.needs_input_grad[1]:
            gtq, gts = mxfp8_quant(gy2.t().contiguous())               # noqa: F821   [N, M], blocks along the tokens
            xtq, xts = mxfp8_quant(x2.t().contiguous())                # noqa: F821   [K, M]
            gw = extra.gemm_mxfp8(gtq, gts, xtq, xts)
        gb = gy2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return gx, gw, gb


# `--fp8-recipe mxfp8` with `--fp8-backward` (or MILES_MXFP8_BACKWARD=1): dgrad and wgrad in MXFP8 too
MXFP8_BACKWARD = os.environ.get("MILES_MXFP8_BACKWARD", "0") == "1"

# `--fp8-recipe mxfp8` (or MILES_MXFP8_LINEAR=1): projections whose K is a multiple of 128 run their forward in MXFP8
MXFP8_LINEAR = os.environ.get("MILES_MXFP8_LINEAR", "0") == "1"


# Inference with pre-quantised weights: the rollout engine registers (payload, scales) for a projection weight; calls
# made without autograd then skip the bf16 weight entirely (half the weight bytes per decode step).
_MXFP8_WEIGHTS: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
MXFP8_MIN_ROWS = 256


def register_mxfp8_weight(w: torch.Tensor, payload: torch.Tensor, scales: torch.Tensor):
    _MXFP8_WEIGHTS[w.data_ptr()] = (payload, scales)


def clear_mxfp8_weights():
    _MXFP8_WEIGHTS.clear()


def linear(x, w, bias=None):
    if x.dtype != BF16:
        return torch.nn.functional.linear(x, w.to(x.dtype), bias)
    if _MXFP8_WEIGHTS and not torch.is_grad_enabled():
        reg = _MXFP8_WEIGHTS.get(w.data_ptr())
        # the block-scaled kernel works on 128×128 tiles: decode-sized batches stay on the split-K bf16 path
        if reg is not None and x.numel() // x.shape[-1] >= MXFP8_MIN_ROWS:
            from . import extra

            y = extra.linear_mxfp8(x, reg[0].view(w.shape), reg[1].view(w.shape[0], -1))
            return y if bias is None else y + bias
    # per-call weight quantisation only pays for itself on training-sized batches: decode-sized calls stay on the bf16 kernels
    if MXFP8_LINEAR and w.dim() == 2 and w.shape[1] % 128 == 0 and w.shape[0] >= 128 and x.numel() // x.shape[-1] >= MXFP8_MIN_ROWS:
        return _LinearMXFP8.apply(x, w, bias)
    return _Linear.apply(x, w, bias)


class _LinearFP32(torch.autograd.Function):
    """y = x·Wᵀ with the fp32 accumulator written out unrounded (router scores, sampling logits)."""

    @staticmethod
    def forward(ctx, x, w):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.save_for_backward(x2, w)
        ctx.shp = shp
        return gemm_nt(x2, w, out_dtype=torch.float32).view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        gy2 = _c(gy.reshape(-1, gy.shape[-1]).to(BF16))
        gx = gemm_nn(gy2, w).view(ctx.shp) if ctx.needs_input_grad[0] else None
        gw = gemm_tn(gy2, x2) if ctx.needs_input_grad[1] else None
        return gx, gw


def linear_fp32(x, w):
    if x.dtype != BF16:
        return torch.nn.functional.linear(x, w.to(x.dtype)).float()
    return _LinearFP32.apply(x, w)


def linear_dgrad(gy, w):
    return gemm_nn(gy, w)


def linear_wgrad(gy, x):
    return gemm_tn(gy, x)


# ---------------------------------------------------------------------------------------------
# norms / activations
# ---------------------------------------------------------------------------------------------

class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x = _c(x)
        y = torch.empty_like(x)
        rstd = torch.empty(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device)
        C.rmsnorm_fwd(x, None, w, y, None, rstd, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, rstd = ctx.saved_tensors
        dx = torch.empty_like(x)
        dw = C.rmsnorm_bwd(x, w, _c(gy), None, rstd, dx)
        return dx, dw, None


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps):
        x, residual = _c(x), _c(residual)
        y = torch.empty_like(x)
        r = torch.empty_like(x)
        rstd = torch.empty(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device)
        C.rmsnorm_fwd(x, residual, w, y, r, rstd, eps)
        ctx.save_for_backward(r, w, rstd)
        return y, r

    @staticmethod
    def backward(ctx, gy, gr):
        r, w, rstd = ctx.saved_tensors
        dx = torch.empty_like(r)
        dw = C.rmsnorm_bwd(r, w, _c(gy), _c(gr) if gr is not None else None, rstd, dx)
        return dx, dx, dw, None


def rmsnorm(x, w, eps=1e-6):
    if x.dtype != BF16:
        return ref.rmsnorm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


def add_rmsnorm(x, residual, w, eps=1e-6):
    if x.dtype != BF16:
        return ref.add_rmsnorm(x, residual, w, eps)
    return _AddRMSNorm.apply(x, residual, w, eps)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        gate_up = _c(gate_up)
        out = torch.empty(*gate_up.shape[:-1], gate_up.shape[-1] // 2, dtype=gate_up.dtype, device=gate_up.device)
        C.swiglu_fwd(gate_up, out, None)
        ctx.save_for_backward(gate_up)
        return out

    @staticmethod
    def backward(ctx, g):
        (gate_up,) = ctx.saved_tensors
        din = torch.empty_like(gate_up)
        C.swiglu_bwd(gate_up, _c(g), din, None)
        return din


def swiglu(gate_up):
    if gate_up.dtype != BF16:
        return ref.swiglu(gate_up)
    return _SwiGLU.apply(gate_up)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, qw, kw, positions, theta, eps):
        T, Hq, D = q.shape
        Hk = k.shape[1]
        assert q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D
        qo = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        ko = torch.empty(T, Hk, D, dtype=k.dtype, device=k.device)
        need = qw is not None
        q_rstd = torch.empty(T * Hq, dtype=torch.float32, device=q.device) if need else None
        k_rstd = torch.empty(T * Hk, dtype=torch.float32, device=q.device) if need else None
        positions = positions.to(torch.int32)
        C.qk_norm_rope_fwd(q, k, qw, kw, positions, qo, ko, q_rstd, k_rstd, theta, eps)
        ctx.save_for_backward(q, k, qw, kw, positions, q_rstd, k_rstd)
        ctx.theta = theta
        return qo, ko

    @staticmethod
    def backward(ctx, gq, gk):
        q, k, qw, kw, positions, q_rstd, k_rstd = ctx.saved_tensors
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dqw = C.qk_norm_rope_bwd(q, qw, q_rstd, _c(gq), positions, dq, ctx.theta)
        dkw = C.qk_norm_rope_bwd(k, kw, k_rstd, _c(gk), positions, dk, ctx.theta)
        return dq, dk, (dqw if qw is not None else None), (dkw if kw is not None else None), None, None, None


def qk_norm_rope(q, k, q_w, k_w, positions, theta, eps=1e-6):
    if q.dtype != BF16 or q.shape[-1] not in (64, 128):
        if q_w is not None:
            q, k = ref.rmsnorm(q, q_w, eps), ref.rmsnorm(k, k_w, eps)
        return ref.rope(q, positions, theta), ref.rope(k, positions, theta)
    return _QKNormRope.apply(q, k, q_w, k_w, positions, float(theta), float(eps))


def qk_norm_rope_cache(q, k, v, q_w, k_w, positions, theta, eps, k_cache, v_cache, slot_mapping):
    """Inference form: norm + rotary on q and k and the KV-cache write of (rotated k, v) in ONE launch.  Returns (q, k)."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    ok = (q.dtype == BF16 and D in (64, 128) and not torch.is_grad_enabled() and q.stride(2) == 1 and q.stride(1) == D
          and k.stride(1) == D and v.stride(1) == D and positions.dtype == torch.int32 and slot_mapping.dtype == torch.int64)
    if not ok:
        q, k = qk_norm_rope(q, k, q_w, k_w, positions, theta, eps)
        kv_cache_write(k, v, k_cache, v_cache, slot_mapping)
        return q, k
    qo = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
    ko = torch.empty(T, Hk, D, dtype=k.dtype, device=k.device)
    publish_limit(LIMIT_KV_SLOTS, k_cache.shape[0] * k_cache.shape[1])
    C.qk_norm_rope_cache(q, k, v, q_w, k_w, positions, qo, ko, k_cache, v_cache, slot_mapping, float(theta), float(eps))
    return qo, ko


class _Rope(torch.autograd.Function):
    """Rotary embedding alone; the backward is the inverse rotation of the incoming gradient."""

    @staticmethod
    def forward(ctx, x, positions, theta, inverse):
        ctx.save_for_backward(positions)
        ctx.theta, ctx.inverse = theta, inverse
        return C.rope(x, positions, float(theta), bool(inverse))

    @staticmethod
    def backward(ctx, g):
        (positions,) = ctx.saved_tensors
        g = g if (g.stride(2) == 1 and g.stride(1) == g.shape[2]) else g.contiguous()
        return C.rope(g, positions, float(ctx.theta), not ctx.inverse), None, None, None


def rope(x, positions, theta, inverse=False):
    if x.dtype != BF16 or x.dim() != 3 or x.shape[-1] not in (64, 128) or x.stride(2) != 1 or x.stride(1) != x.shape[2]:
        return ref.rope(x, positions, theta, inverse)
    return _Rope.apply(x, positions.to(torch.int32), theta, inverse)


def kv_cache_write(k, v, k_cache, v_cache, slot_mapping):
    assert k.stride(2) == 1 and k.stride(1) == k.shape[2]
    publish_limit(LIMIT_KV_SLOTS, k_cache.shape[0] * k_cache.shape[1])
    C.kv_cache_write(k.detach(), v.detach(), k_cache, v_cache, slot_mapping.to(torch.int64))


# ---------------------------------------------------------------------------------------------
# optimizer
# ---------------------------------------------------------------------------------------------

def adamw_step_masked(master, grad, exp_avg, exp_avg_sq, decay_mask, lr, b1, b2, eps, wd, step, scale, param_out):
    if not torch.is_tensor(scale):
        scale = torch.tensor([float(scale)], dtype=torch.float32, device=master.device)
    else:
        scale = scale.reshape(1).float()
    C.adamw(master, grad, exp_avg, exp_avg_sq, decay_mask, scale, param_out, lr, b1, b2, eps, wd, step)


def adamw_step(master, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, param_out=None):
    adamw_step_masked(master, grad.float(), exp_avg, exp_avg_sq, None, lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                      param_out)


from .cuda_more import *  # noqa: E402,F401,F403  (attention, MoE, log-prob, sampling, quantisation)
