"""Sparse attention families: lightning indexer + top-k sparse attention (DSA), pooled-key selection (k-pool), and
per-query index-list / block-sparse attention (QSA).

Reference kernels: miles/kernels/attention/dsa/tilelang/indexer_fwd.py:8-140, indexer_bwd.py:18-165,
sparse_attention_fwd.py:9-207, sparse_attention_bwd.py:10-301, dsa/sparse_attention.py:1-182, dsa/kpool.py:21-250,
qsa/sparse_attention.py:14-280, qsa/block_sparse_attention.py:16-579.

Shapes are packed-token ("thd"): q [T, H, D], k [Tkv, Hk, D], v [Tkv, Hk, Dv]; an index list row holds key positions
(global rows of k/v) with −1 padding.  MLA-style models pass Hk = 1 (one shared latent key/value per token).
Every function is a differentiable fp32 PyTorch statement (the CPU path and the oracle); `sparse_attention` has a
one-pass CUDA forward (`ops/csrc/sparse_attn.cu`: one warp per (query, head), online softmax over the gathered keys)
used when gradients are off, i.e. in the rollout engine.
"""
from __future__ import annotations

import math

import torch


# ---- DSA: lightning indexer ----------------------------------------------------------------------------------------

def lightning_indexer(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, q_pos: torch.Tensor | None = None,
                      k_pos: torch.Tensor | None = None, q_seq: torch.Tensor | None = None, k_seq: torch.Tensor | None = None) -> torch.Tensor:
    """logits[t, s] = Σ_h w[t, h] · relu(q_idx[t, h] · k_idx[s]);  −inf where s is not visible from t
    (another sequence, or later in the same one).  q_idx [T, Hi, Di], k_idx [Tkv, Di], w [T, Hi]."""
    s = torch.einsum("thd,sd->ths", q_idx.float(), k_idx.float())
    logits = (torch.relu(s) * w.float().unsqueeze(-1)).sum(1)
    mask = visibility_mask(q_idx.shape[0], k_idx.shape[0], q_pos, k_pos, q_seq, k_seq, q_idx.device)
    return logits.masked_fill(~mask, float("-inf"))


def visibility_mask(T, Tkv, q_pos, k_pos, q_seq, k_seq, device) -> torch.Tensor:
    if q_pos is None:
        q_pos, k_pos = torch.arange(T, device=device) + (Tkv - T), torch.arange(Tkv, device=device)
    m = k_pos.view(1, -1) <= q_pos.view(-1, 1)
    if q_seq is not None:
        m &= q_seq.view(-1, 1) == k_seq.view(1, -1)
    return m


def indexer_topk(logits: torch.Tensor, topk: int) -> torch.Tensor:
    """Indices of the top-k visible keys per query, −1 where fewer than k are visible.  int32 [T, topk]."""
    k = min(topk, logits.shape[1])
    val, idx = logits.topk(k, dim=-1)
    idx = torch.where(torch.isfinite(val), idx, torch.full_like(idx, -1))
    if k < topk:
        idx = torch.cat([idx, idx.new_full((idx.shape[0], topk - k), -1)], -1)
    return idx.to(torch.int32)


# ---- sparse attention over an index list ------------------------------------------------------------------------------

def sparse_attention_ref(q, k, v, indices, scale: float | None = None, sink: torch.Tensor | None = None):
    """out[t, h] = softmax_j(scale · q[t, h]·k[idx[t, j], hk])ᵀ v[idx[t, j], hk]  (+ a per-head sink logit in the
    denominator).  Returns (out [T, H, Dv] in q's dtype, lse fp32 [T, H])."""
    T, H, D = q.shape
    Hk, Dv = k.shape[1], v.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    valid = indices >= 0
    idx = indices.clamp_min(0).long()
    kg = k.float()[idx]                                   # [T, K, Hk, D]
    vg = v.float()[idx]
    rep = H // Hk
    kg = kg.repeat_interleave(rep, dim=2)                 # [T, K, H, D]
    vg = vg.repeat_interleave(rep, dim=2)
    s = torch.einsum("thd,tkhd->thk", q.float(), kg) * scale
    s = s.masked_fill(~valid.unsqueeze(1), float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.float().view(1, H, 1).expand(T, H, 1)], -1)
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)                      # rows with no visible key and no sink
    if sink is not None:
        p = p[..., :-1]
    out = torch.einsum("thk,tkhd->thd", p, vg)
    return out.to(q.dtype), lse


def sparse_attention(q, k, v, indices, scale: float | None = None, sink: torch.Tensor | None = None):
    D, Dv = q.shape[-1], v.shape[-1]
    if (q.is_cuda and not torch.is_grad_enabled() and q.dtype == torch.bfloat16 and D % 32 == 0 and Dv % 32 == 0
            and D <= 576 and Dv <= 512 and q.shape[1] % k.shape[1] == 0):
        from . import cuda

        T, H, _ = q.shape
        out = torch.empty(T, H, Dv, dtype=q.dtype, device=q.device)
        lse = torch.empty(T, H, dtype=torch.float32, device=q.device)
        cuda.C.sparse_attention_fwd(q.contiguous(), k.contiguous(), v.contiguous(), indices.to(torch.int32).contiguous(),
                                    sink.float().contiguous() if sink is not None else None, out, lse,
                                    float(scale if scale is not None else 1.0 / math.sqrt(D)))
        return out, lse
    return sparse_attention_ref(q, k, v, indices, scale, sink)


def dsa_attention(q, k, v, q_idx, k_idx, w_idx, topk: int, scale=None, sink=None, q_seq=None, k_seq=None, q_pos=None, k_pos=None):
    """DeepSeek-style sparse attention: the lightning indexer picks `topk` keys per query, attention runs over them."""
    logits = lightning_indexer(q_idx, k_idx, w_idx, q_pos, k_pos, q_seq, k_seq)
    idx = indexer_topk(logits.detach(), topk)
    out, lse = sparse_attention(q, k, v, idx, scale, sink)
    return out, idx, logits


def indexer_kl_loss(logits: torch.Tensor, attn_probs_sum: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Training signal of the indexer: KL(target ‖ softmax(indexer logits)) on the selected keys, where the target is
    the main attention's probability mass per key summed over heads (detached) and renormalised."""
    valid = indices >= 0
    sel = logits.gather(1, indices.clamp_min(0).long()).masked_fill(~valid, float("-inf"))
    logp = torch.log_softmax(sel, -1)
    tgt = attn_probs_sum.detach() * valid
    tgt = tgt / tgt.sum(-1, keepdim=True).clamp_min(1e-20)
    return (tgt * (torch.log(tgt.clamp_min(1e-20)) - logp.masked_fill(~valid, 0.0))).sum(-1).mean()


# ---- k-pool: pooled-key selection ------------------------------------------------------------------------------------

def pooled_keys(k: torch.Tensor, block: int) -> torch.Tensor:
    """Mean of every `block` consecutive keys (the last block may be short).  k [Tkv, D] → [ceil(Tkv/block), D]."""
    Tkv, D = k.shape
    nb = (Tkv + block - 1) // block
    pad = nb * block - Tkv
    kp = torch.cat([k.float(), k.new_zeros(pad, D, dtype=torch.float32)]) if pad else k.float()
    cnt = torch.full((nb, 1), float(block), device=k.device)
    if pad:
        cnt[-1] = block - pad
    return kp.view(nb, block, D).sum(1) / cnt


def kpool_select(q: torch.Tensor, k: torch.Tensor, block: int, top_blocks: int, tail: int = 0) -> torch.Tensor:
    """Per query (positions aligned to the end of k): score key blocks by q·mean(k_block), keep the `top_blocks` best
    fully-visible blocks, expand them to token indices and append the `tail` most recent tokens.  int32 [T, top_blocks·block + tail]."""
    T, Tkv = q.shape[0], k.shape[0]
    pk = pooled_keys(k, block)
    nb = pk.shape[0]
    q_pos = torch.arange(T, device=q.device) + (Tkv - T)
    scores = q.float() @ pk.t()
    blk_end = (torch.arange(nb, device=q.device) + 1) * block - 1
    visible = blk_end.view(1, -1) <= (q_pos.view(-1, 1) - tail)          # whole block before the tail window
    scores = scores.masked_fill(~visible, float("-inf"))
    kb = min(top_blocks, nb)
    val, bidx = scores.topk(kb, dim=-1)
    tok = bidx.unsqueeze(-1) * block + torch.arange(block, device=q.device)
    tok = torch.where(torch.isfinite(val).unsqueeze(-1), tok, torch.full_like(tok, -1)).reshape(T, kb * block)
    if kb < top_blocks:
        tok = torch.cat([tok, tok.new_full((T, (top_blocks - kb) * block), -1)], -1)
    if tail:
        t_idx = q_pos.view(-1, 1) - torch.arange(tail - 1, -1, -1, device=q.device).view(1, -1)
        tok = torch.cat([tok, torch.where(t_idx >= 0, t_idx, torch.full_like(t_idx, -1))], -1)
    return tok.to(torch.int32)


# ---- QSA: block-sparse attention ----------------------------------------------------------------------------------------

def block_sparse_attention(q, k, v, block_indices: torch.Tensor, block_size: int, scale: float | None = None, causal: bool = True):
    """Each query attends to the key blocks listed in `block_indices` [T, nb] (−1 padded); inside the diagonal block the
    causal mask applies token by token.  Positions of q are aligned to the end of k."""
    T, Tkv = q.shape[0], k.shape[0]
    tok = block_indices.unsqueeze(-1).long() * block_size + torch.arange(block_size, device=q.device)
    tok = torch.where((block_indices >= 0).unsqueeze(-1), tok, torch.full_like(tok, -1)).reshape(T, -1)
    tok = torch.where(tok < Tkv, tok, torch.full_like(tok, -1))
    if causal:
        q_pos = (torch.arange(T, device=q.device) + (Tkv - T)).view(-1, 1)
        tok = torch.where(tok <= q_pos, tok, torch.full_like(tok, -1))
    return sparse_attention(q, k, v, tok.to(torch.int32), scale)
