"""Second half of the CUDA op layer: attention, MoE, log-prob head, sampling, quantisation."""
from __future__ import annotations

import math
import os

import torch

from . import reference as ref
from .cuda import BF16, LIMIT_KV_BLOCKS, LIMIT_MOE_PAIRS, C, _c, gemm_nn, gemm_nt, gemm_tn, publish_limit

# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------


USE_TC_ATTENTION = os.environ.get("MILES_TC_ATTENTION", "1") != "0"
USE_TC_ATTENTION_BWD = os.environ.get("MILES_TC_ATTENTION_BWD", "1") != "0"


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal):
        T, Hq, D = q.shape
        assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D and v.stride(2) == 1
        scale = 1.0 / math.sqrt(D)
        o = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
        if T > 0 and cu_seqlens.numel() > 1:
            if max_seqlen <= 0:
                max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
            if D == 128 and USE_TC_ATTENTION and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0:
                # tcgen05 forward (TMA-fed, accumulators in tensor memory)
                C.flash_fwd_tc(q, k, v, o, lse, cu_seqlens, max_seqlen, scale, causal, C.error_flag(q), None)
            else:
                C.flash_fwd(q, k, v, o, lse, cu_seqlens, max_seqlen, scale, causal)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.max_seqlen, ctx.causal, ctx.scale = max_seqlen, causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu = ctx.saved_tensors
        do = _c(do)
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        delta = torch.empty_like(lse)
        D = q.shape[-1]
        if (D == 128 and USE_TC_ATTENTION_BWD and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0
                and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D):
            # tcgen05 backward: Sᵀ/dPᵀ and the dK, dV, dQ accumulators live in tensor memory
            C.flash_bwd_tc(q, k, v, o, do, lse, delta, dq, dk, dv, cu, ctx.max_seqlen, ctx.scale, ctx.causal, C.error_flag(q))
        else:
            C.flash_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, cu, ctx.max_seqlen, ctx.scale, ctx.causal)
        return dq, dk, dv, None, None, None


def attention_varlen(q, k, v, cu_seqlens, max_seqlen=0, causal=True):
    if q.dtype != BF16 or q.shape[-1] not in (64, 128):
        return ref.attention_varlen(q, k, v, cu_seqlens, causal)
    return _FlashAttn.apply(q, k, v, cu_seqlens.to(torch.int32), int(max_seqlen), bool(causal))


_DECODE_SPLITS = int(os.environ.get("MILES_DECODE_SPLITS", "8"))   # KV splits per (request, kv head) in paged decode


def extend_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens, extend=None):
    """New tokens of each request attend to that request's whole paged KV (which already contains them): the keys and
    values are gathered from the cache into packed buffers and the tcgen05 forward kernel runs with separate query and key
    sequences — query i of a request sees keys ≤ i + (Lk − Lq)."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    if extend is None:                       # callers outside the engine: build the description here (host round trip)
        bs = k_cache.shape[1]
        sl, ql = seq_lens.tolist(), q_lens.tolist()
        slots = [int(block_table[b, p // bs]) * bs + p % bs for b, L in enumerate(sl) for p in range(L)]
        cu_q = torch.tensor([0] + list(torch.tensor(ql).cumsum(0).tolist()), dtype=torch.int32, device=q.device)
        cu_k = torch.tensor([0] + list(torch.tensor(sl).cumsum(0).tolist()), dtype=torch.int32, device=q.device)
        extend = {"cu_q": cu_q, "cu_k": cu_k, "kv_slots": torch.tensor(slots, dtype=torch.int64, device=q.device), "max_k": max(sl)}
    kk = k_cache.view(-1, Hkv, D).index_select(0, extend["kv_slots"])
    vv = v_cache.view(-1, Hkv, D).index_select(0, extend["kv_slots"])
    max_q = int(q_lens.max().item()) if "max_q" not in extend else extend["max_q"]
    if q.dtype != BF16 or D != 128 or not USE_TC_ATTENTION:
        return ref.paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens=q_lens)
    q = _c(q)
    o = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    C.flash_fwd_tc(q, kk, vv, o, lse, extend["cu_q"], max_q, 1.0 / math.sqrt(D), True, C.error_flag(q), extend["cu_k"])
    return o


def paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens=None, max_q_len=1, extend=None):
    """Decode (one new token per request) over the paged cache; with `q_lens` a prefill that continues cached KV
    (`extend_attention`)."""
    if q_lens is not None:
        if extend is not None:
            extend = dict(extend, max_q=int(max_q_len))
        return extend_attention(q, k_cache, v_cache, block_table, seq_lens, q_lens, extend)
    B, Hq, D = q.shape
    group = Hq // k_cache.shape[2]
    if q.dtype != BF16 or D not in (64, 128) or group not in (1, 2, 4, 8):
        return ref.paged_attention(q, k_cache, v_cache, block_table, seq_lens)
    q = _c(q)
    out = torch.empty_like(q)
    # enough (request, kv head, split) CTAs for two waves of the 148 SMs, never more splits than that needs
    splits = max(1, min(_DECODE_SPLITS, -(-296 // (B * k_cache.shape[2]))))
    part_o = torch.empty(B * Hq * splits * D, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=q.device)
    publish_limit(LIMIT_KV_BLOCKS, k_cache.shape[0])
    C.paged_decode(q, k_cache, v_cache, block_table, seq_lens, out, part_o, part_ml, 1.0 / math.sqrt(D), splits)
    return out


# ---------------------------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------------------------

class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, normalize):
        w, idx, probs = C.router_topk(_c(logits.float()), k, normalize, True)
        ctx.save_for_backward(probs, idx, w)
        ctx.normalize = normalize
        ctx.mark_non_differentiable(idx)
        return w, idx, probs

    @staticmethod
    def backward(ctx, gw, _gidx, gprobs):
        probs, idx, w = ctx.saved_tensors
        li = idx.long()
        gw = gw.float()
        if ctx.normalize:
            # w_j = p_j / S, S = Σ_sel p  ⇒  dL/dp_j = (g_j − Σ_i g_i w_i) / S
            S = probs.gather(1, li).sum(-1, keepdim=True).clamp_min(1e-20)
            gp_sel = (gw - (gw * w).sum(-1, keepdim=True)) / S
        else:
            gp_sel = gw
        gp = torch.zeros_like(probs).scatter_add_(1, li, gp_sel)
        if gprobs is not None:
            gp = gp + gprobs
        # softmax backward
        gl = probs * (gp - (gp * probs).sum(-1, keepdim=True))
        return gl, None, None


def router_topk(logits, k, normalize=True):
    if logits.shape[-1] > 256:
        return ref.router_topk(logits, k, normalize)
    return _RouterTopK.apply(logits, int(k), bool(normalize))


# ---------------------------------------------------------------------------------------------
# MoE FFN (single rank or the local part of an expert-parallel layer)
# ---------------------------------------------------------------------------------------------

def moe_max_rows(n_pairs: int, num_experts: int) -> int:
    """Worst-case padded row count: every expert's segment rounded up to 128."""
    return (n_pairs + num_experts * 127 + 127) // 128 * 128


# Inference with few tokens per expert (decode): segments are padded to 16/32/64 rows instead of 128 and the grouped
# GEMMs run with the expert weights on the 128-row MMA side (gemm_small.cu).  MILES_SMALL_MOE=0 turns the path off.
SMALL_MOE_AVG = float(os.environ.get("MILES_SMALL_MOE_AVG", "32")) if os.environ.get("MILES_SMALL_MOE", "1") != "0" else 0.0


MOE_GEMV_T = min(8, int(os.environ.get("MILES_MOE_GEMV_T", "8")))


def small_moe_bt(n_pairs: int, num_experts: int, w13, w2) -> int:
    """Row granularity for an inference MoE call: 128 (general path) or a decode-sized tile."""
    if SMALL_MOE_AVG <= 0 or torch.is_grad_enabled() or w13.shape[1] % 128 or w2.shape[1] % 128:
        return 128
    avg = n_pairs / max(num_experts, 1)
    if avg > SMALL_MOE_AVG:
        return 128
    return 16 if avg <= 16 else 32          # measured: the finest tile wins (weight re-reads hit L2, padding rows do not)


def moe_max_rows_pad(n_pairs: int, num_experts: int, pad: int) -> int:
    return (n_pairs + num_experts * (pad - 1) + pad - 1) // pad * pad


def experts_forward(x_perm, w13, w2, seg, tile, bt: int = 128):
    """Grouped expert FFN on expert-sorted rows whose segments are padded to `bt`. Returns (h1 pre-activation, y_perm)."""
    max_rows, H = x_perm.shape
    E, F2, _ = w13.shape
    h1 = torch.empty(max_rows, F2, dtype=x_perm.dtype, device=x_perm.device)
    act = torch.empty(max_rows, F2 // 2, dtype=x_perm.dtype, device=x_perm.device)
    y_perm = torch.empty(max_rows, H, dtype=x_perm.dtype, device=x_perm.device)
    if bt != 128:
        C.gemm_small_grouped(x_perm, w13, h1, max_rows, F2, H, E, tile, seg[-1:], bt)
        C.swiglu_fwd(h1, act, seg[-1:])
        C.gemm_small_grouped(act, w2, y_perm, max_rows, H, F2 // 2, E, tile, seg[-1:], bt)
        return h1, y_perm
    from . import cuda as _cuda

    if _cuda.MXFP8_LINEAR and H % 128 == 0 and F2 % 256 == 0 and max_rows >= 8 * _cuda.MXFP8_MIN_ROWS:
        # --fp8-recipe mxfp8: the expert GEMMs of the forward run block-scaled (activations quantised per call, expert weights
        # once per call); the backward uses the bf16 grouped GEMMs on the unquantised operands (straight-through), like the
        # dense projections of this recipe
        from . import extra

        F = F2 // 2
        xq, xs = mxfp8_quant(x_perm)
        wq, ws = mxfp8_quant(w13.reshape(E * F2, H))
        extra.gemm_mxfp8_grouped(xq, xs, wq.view(E, F2, H), ws.view(E, F2, H // 32), tile, out=h1)
        C.swiglu_fwd(h1, act, seg[-1:])
        aq, as_ = mxfp8_quant(act)
        w2q, w2s = mxfp8_quant(w2.reshape(E * H, F))
        extra.gemm_mxfp8_grouped(aq, as_, w2q.view(E, H, F), w2s.view(E, H, F // 32), tile, out=y_perm)
        return h1, y_perm
    C.gemm_grouped(x_perm, w13, h1, max_rows, F2, H, E, tile, False, 0)
    C.swiglu_fwd(h1, act, seg[-1:])
    C.gemm_grouped(act, w2, y_perm, max_rows, H, F2 // 2, E, tile, False, 0)
    return h1, y_perm


def _moe_ffn_small(x, w13, w2, topk_w, topk_idx, expert_offset, bt):
    T, H = x.shape
    E = w13.shape[0]
    k = topk_idx.shape[1]
    x = _c(x)
    idx32 = _c(topk_idx.to(torch.int32)).view(-1)
    max_rows = moe_max_rows_pad(T * k, E, bt)
    seg, tile, row_src, dst_row = C.moe_align(idx32, E, expert_offset, max_rows, None, bt)
    x_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
    publish_limit(LIMIT_MOE_PAIRS, x.shape[0] * k)
    C.moe_gather(x, x_perm, row_src, seg, k)
    _, y_perm = experts_forward(x_perm, _c(w13), _c(w2), seg, tile, bt)
    out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    C.moe_combine(y_perm, _c(topk_w.float()), dst_row, out, k)
    return out


def experts_backward(dy_perm, x_perm, h1, w13, w2, seg, tile):
    """Backward of `experts_forward`: returns (dx_perm, dw13, dw2)."""
    max_rows, H = x_perm.shape
    E, F2, _ = w13.shape
    F = F2 // 2
    dt, dev = x_perm.dtype, x_perm.device
    act = torch.empty(max_rows, F, dtype=dt, device=dev)
    C.swiglu_fwd(h1, act, seg[-1:])
    dact = torch.empty(max_rows, F, dtype=dt, device=dev)
    C.gemm_grouped(dy_perm, w2, dact, max_rows, F, H, E, tile, True, 0)
    dw2 = torch.empty_like(w2)
    C.gemm_grouped_wgrad(dy_perm, act, dw2, max_rows, H, F, E, seg, False, 0)
    dh1 = torch.empty(max_rows, F2, dtype=dt, device=dev)
    C.swiglu_bwd(h1, dact, dh1, seg[-1:])
    dw13 = torch.empty_like(w13)
    C.gemm_grouped_wgrad(dh1, x_perm, dw13, max_rows, F2, H, E, seg, False, 0)
    dx_perm = torch.empty(max_rows, H, dtype=dt, device=dev)
    C.gemm_grouped(dh1, w13, dx_perm, max_rows, H, F2, E, tile, True, 0)
    return dx_perm, dw13, dw2


class _MoEFFN(torch.autograd.Function):
    """y[t] = Σ_j w[t,j] · W2[e]·swiglu(W13[e]·x[t]) with e = idx[t,j] − expert_offset ∈ [0, E_local) (others skipped)."""

    @staticmethod
    def forward(ctx, x, w13, w2, topk_w, topk_idx, expert_offset):
        T, H = x.shape
        E, F2, _ = w13.shape
        F = F2 // 2
        k = topk_idx.shape[1]
        x = _c(x)
        idx32 = _c(topk_idx.to(torch.int32)).view(-1)
        wf = _c(topk_w.float())
        max_rows = moe_max_rows(T * k, E)
        seg, tile, row_src, dst_row = C.moe_align(idx32, E, expert_offset, max_rows, None)
        x_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
        publish_limit(LIMIT_MOE_PAIRS, x.shape[0] * k)
        C.moe_gather(x, x_perm, row_src, seg, k)
        h1, y_perm = experts_forward(x_perm, w13, w2, seg, tile)        # bf16 grouped GEMMs, or block-scaled under the MXFP8 recipe
        out = torch.empty(T, H, dtype=x.dtype, device=x.device)
        C.moe_combine(y_perm, wf, dst_row, out, k)
        ctx.save_for_backward(x, w13, w2, wf, seg, tile, row_src, dst_row, h1, y_perm)
        ctx.k = k
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w13, w2, wf, seg, tile, row_src, dst_row, h1, y_perm = ctx.saved_tensors
        k = ctx.k
        T, H = x.shape
        E, F2, _ = w13.shape
        F = F2 // 2
        max_rows = h1.shape[0]
        dout = _c(dout)
        dy_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
        dw_flat = torch.zeros(T * k, dtype=torch.float32, device=x.device)
        C.moe_combine_bwd(dout, y_perm, wf.view(-1), row_src, seg, dy_perm, dw_flat, k)
        # through W2: dact = dy_perm · W2 ; dW2[e] = dy_permᵀ · act
        act = torch.empty(max_rows, F, dtype=x.dtype, device=x.device)
        C.swiglu_fwd(h1, act, seg[-1:])
        dact = torch.empty(max_rows, F, dtype=x.dtype, device=x.device)
        C.gemm_grouped(dy_perm, w2, dact, max_rows, F, H, E, tile, True, 0)
        dw2 = torch.empty_like(w2)
        C.gemm_grouped_wgrad(dy_perm, act, dw2, max_rows, H, F, E, seg, False, 0)
        dh1 = torch.empty(max_rows, F2, dtype=x.dtype, device=x.device)
        C.swiglu_bwd(h1, dact, dh1, seg[-1:])
        x_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
        publish_limit(LIMIT_MOE_PAIRS, x.shape[0] * k)
        C.moe_gather(x, x_perm, row_src, seg, k)
        dw13 = torch.empty_like(w13)
        C.gemm_grouped_wgrad(dh1, x_perm, dw13, max_rows, F2, H, E, seg, False, 0)
        dx_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
        C.gemm_grouped(dh1, w13, dx_perm, max_rows, H, F2, E, tile, True, 0)
        dx = torch.empty_like(x)
        C.moe_combine(dx_perm, None, dst_row, dx, k)
        return dx, dw13, dw2, dw_flat.view(T, k), None, None


def moe_ffn(x, w13, w2, topk_w, topk_idx, expert_offset: int = 0):
    if x.dtype != BF16:
        return ref.moe_ffn(x, w13, w2, topk_w, topk_idx)
    T, k = topk_idx.shape
    if (0 < T <= MOE_GEMV_T and T * k <= 64 and not torch.is_grad_enabled() and x.shape[1] % 32 == 0
            and w13.shape[1] % 64 == 0
            # both kernels keep their activations in shared memory next to a 64 KB weight ring
            and 65536 + max(8 * (2 * x.shape[1] + 64), T * k * (w13.shape[1] + 64)) <= 200 * 1024):
        # a handful of tokens: two matrix-vector kernels, no sort / gather / combine (gemv.cu)
        act = torch.empty(T * k, w13.shape[1] // 2, dtype=x.dtype, device=x.device)
        out = torch.empty_like(x)
        C.moe_gemv(_c(x), _c(w13), _c(w2), _c(topk_idx.to(torch.int32)), _c(topk_w.float()), act, out, int(expert_offset))
        return out
    bt = small_moe_bt(topk_idx.numel(), w13.shape[0], w13, w2)
    if bt != 128 and x.shape[0]:
        return _moe_ffn_small(x, w13, w2, topk_w, topk_idx, int(expert_offset), bt)
    return _MoEFFN.apply(x, w13, w2, topk_w, topk_idx, int(expert_offset))


# ---------------------------------------------------------------------------------------------
# log-prob / entropy head: vocabulary streamed in chunks, logits never materialised in full
# ---------------------------------------------------------------------------------------------
_VOCAB_CHUNK = 16384
_ROW_CHUNK = 16384


def _vocab_chunks(V):
    return [(v0, min(V, v0 + _VOCAB_CHUNK)) for v0 in range(0, V, _VOCAB_CHUNK)]


class _LogProbEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, w, targets, temperature, with_entropy, vocab_offset):
        R, H = hidden.shape
        V = w.shape[0]
        hidden = _c(hidden)
        tg = _c(targets.to(torch.int64)) - vocab_offset
        inv_t = 1.0 / temperature
        logp = torch.empty(R, dtype=torch.float32, device=hidden.device)
        ent = torch.empty(R, dtype=torch.float32, device=hidden.device)
        lse = torch.empty(R, dtype=torch.float32, device=hidden.device)
        for r0 in range(0, R, _ROW_CHUNK):
            r1 = min(R, r0 + _ROW_CHUNK)
            stats = torch.empty(r1 - r0, 4, dtype=torch.float32, device=hidden.device)
            for ci, (v0, v1) in enumerate(_vocab_chunks(V)):
                logits = gemm_nt(hidden[r0:r1], w[v0:v1], out_dtype=torch.float32)
                C.logit_stats(logits, tg[r0:r1], stats, v0, inv_t, ci == 0)
            C.logit_stats_finish(stats, logp[r0:r1], ent[r0:r1], lse[r0:r1])
        ctx.save_for_backward(hidden, w, tg, lse, ent)
        ctx.inv_t, ctx.with_entropy = inv_t, with_entropy
        ctx.mark_non_differentiable(lse)
        return logp, ent, lse

    @staticmethod
    def backward(ctx, g_lp, g_ent, _g_lse):
        hidden, w, tg, lse, ent = ctx.saved_tensors
        R, H = hidden.shape
        V = w.shape[0]
        g_lp = _c(g_lp.float()) if g_lp is not None else None
        g_ent = _c(g_ent.float()) if (g_ent is not None and ctx.with_entropy) else None
        dh = torch.zeros(R, H, dtype=torch.float32, device=hidden.device)
        dw = torch.empty_like(w)
        for (v0, v1) in _vocab_chunks(V):
            dwc = None
            for r0 in range(0, R, _ROW_CHUNK):
                r1 = min(R, r0 + _ROW_CHUNK)
                logits = gemm_nt(hidden[r0:r1], w[v0:v1], out_dtype=torch.float32)
                dl = torch.empty(r1 - r0, v1 - v0, dtype=BF16, device=hidden.device)
                C.logit_grad(logits, tg[r0:r1], lse[r0:r1], ent[r0:r1] if g_ent is not None else None,
                             g_lp[r0:r1] if g_lp is not None else None, g_ent[r0:r1] if g_ent is not None else None, dl, v0,
                             ctx.inv_t)
                # dH[r0:r1] += dl · W_c   (fp32 accumulate in place)
                Mr, Kc, Nh = r1 - r0, v1 - v0, H
                C.gemm(dl, w[v0:v1], dh[r0:r1], Mr, Nh, Kc, Kc, Nh, H, False, True, True, None, 0)
                # dW_c (+)= dlᵀ · H
                if dwc is None:
                    dwc = torch.empty(v1 - v0, H, dtype=torch.float32, device=hidden.device) if R > _ROW_CHUNK else dw[v0:v1]
                    gemm_tn(dl, hidden[r0:r1], out=dwc)
                else:
                    gemm_tn(dl, hidden[r0:r1], out=dwc, accumulate=True)
            if dwc.dtype != dw.dtype:
                dw[v0:v1].copy_(dwc)
        return dh.to(hidden.dtype), dw, None, None, None, None


def logprob_entropy(hidden, w, targets, temperature=1.0, with_entropy=False, vocab_offset: int = 0, return_lse=False):
    if hidden.dtype != BF16:
        lp, ent = ref.logprob_entropy(hidden, w, targets, temperature, with_entropy=with_entropy)
        return lp, ent
    logp, ent, lse = _LogProbEntropy.apply(hidden, w, targets, float(temperature), bool(with_entropy), int(vocab_offset))
    if return_lse:
        return logp, ent, lse
    return logp, (ent if with_entropy else None)


# ---------------------------------------------------------------------------------------------
# sampling / quantisation
# ---------------------------------------------------------------------------------------------

def sample_logprob(logits, temperature, greedy, seeds=None, step: int = 0):
    logits = _c(logits.float())
    return tuple(C.sample_logprob(logits, _c(temperature.float()), _c(greedy.to(torch.uint8)),
                                  _c(seeds.to(torch.int64)) if seeds is not None else None, int(step)))


def mxfp8_quant(x):
    assert x.dtype == BF16 and x.shape[-1] % 32 == 0
    q, s = C.mxfp8_quant(_c(x))
    return q, s


def fp8_blockwise_quant(w):
    assert w.dtype == BF16 and w.dim() == 2
    q, s = C.fp8_block_quant(_c(w))
    return q, s


def int4_fake_quant(x, block_m=1, block_n=32, symmetric=True):
    assert x.dtype == BF16 and x.dim() == 2
    y, s = C.int4_fake_quant(_c(x), block_m, block_n, symmetric)
    return y, s


def absmax(x):
    return C.absmax(_c(x))


def nvfp4_qdq(x, global_amax=None, four_over_six=False):
    assert x.dtype == BF16 and x.numel() % 16 == 0
    x = _c(x)
    if global_amax is None:
        global_amax = C.absmax(x)
    return C.nvfp4_qdq(x, global_amax.reshape(1).float(), bool(four_over_six))
