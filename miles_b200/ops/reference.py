"""Plain-PyTorch statements of every op the CUDA extension implements.

They are the CPU execution path (tests without a GPU, the gloo plumbing run) and the numerical
oracle for the sm_100a kernels: each kernel test compares against these evaluated in fp32.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------------------------
# normalisation / activation / position
# --------------------------------------------------------------------------------------------

def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """residual' = residual + x ; y = rmsnorm(residual').  Returns (y, residual')."""
    r = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(r, w, eps), r


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up [..., 2F] with gate in the first half → silu(gate) * up."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, inverse: bool = False) -> torch.Tensor:
    """NeoX-style rotary embedding on x [T, heads, head_dim] (pairs are (i, i + d/2))."""
    d = x.shape[-1]
    cos, sin = rope_cos_sin(positions, d, theta)
    if inverse:
        sin = -sin
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


# --------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------

def router_topk(logits: torch.Tensor, k: int, normalize: bool = True):
    """Softmax over all experts (fp32) → top-k → optional renormalisation.

    Returns (weights fp32 [T,k], indices int32 [T,k], probs fp32 [T,E]).
    Ties are broken toward the lower expert id so that train and rollout agree.
    """
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1, sorted=True)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w, idx.to(torch.int32), probs


def gather_router_weights(probs: torch.Tensor, idx: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """Routing replay: weights re-gathered from *current* probabilities at recorded indices."""
    w = probs.gather(1, idx.long())
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------

def attention_varlen(q, k, v, cu_seqlens: torch.Tensor, causal: bool = True, scale: float | None = None):
    """Packed (THD) causal attention with GQA.  q [T,Hq,D], k/v [T,Hkv,D]; cu_seqlens int32 [B+1]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e == s:
            continue
        qb = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        kb = k[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vb = v[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        sc = torch.matmul(qb, kb.transpose(1, 2)) * scale
        if causal:
            L = e - s
            m = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            sc = sc.masked_fill(~m, float("-inf"))
        p = torch.softmax(sc, dim=-1)
        out[s:e] = torch.matmul(p, vb).transpose(0, 1).to(q.dtype)
    return out


def paged_attention(q, k_cache, v_cache, block_table, seq_lens, scale: float | None = None, q_lens=None):
    """Attention of new query tokens over a paged KV cache (decode and chunked prefill).

    q [T,Hq,D] packed by request (q_lens per request, default all ones);
    k_cache/v_cache [num_blocks, block_size, Hkv, D]; block_table int32 [B, max_blocks];
    seq_lens int32 [B] = KV length *including* the new tokens (already written to the cache).
    Query token j (0-based among the request's q_len new tokens) sees keys [0, seq_len - q_len + j].
    """
    B = block_table.shape[0]
    Hq, D = q.shape[1], q.shape[2]
    bs = k_cache.shape[1]
    Hkv = k_cache.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    if q_lens is None:
        q_lens = [1] * B
    else:
        q_lens = q_lens.tolist() if torch.is_tensor(q_lens) else list(q_lens)
    sl = seq_lens.tolist()
    off = 0
    for b in range(B):
        L, ql = sl[b], q_lens[b]
        if ql == 0:
            continue
        nb = (L + bs - 1) // bs
        blocks = block_table[b, :nb].long()
        kb = k_cache[blocks].reshape(nb * bs, Hkv, D)[:L].float().transpose(0, 1).repeat_interleave(g, 0)
        vb = v_cache[blocks].reshape(nb * bs, Hkv, D)[:L].float().transpose(0, 1).repeat_interleave(g, 0)
        qb = q[off:off + ql].float().transpose(0, 1)  # [Hq, ql, D]
        sc = torch.matmul(qb, kb.transpose(1, 2)) * scale  # [Hq, ql, L]
        pos_q = torch.arange(L - ql, L, device=q.device)[:, None]
        pos_k = torch.arange(L, device=q.device)[None, :]
        sc = sc.masked_fill(pos_k > pos_q, float("-inf"))
        p = torch.softmax(sc, dim=-1)
        out[off:off + ql] = torch.matmul(p, vb).transpose(0, 1).to(q.dtype)
        off += ql
    return out


# --------------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------------

def moe_ffn(x, w13, w2, topk_w, topk_idx):
    """x [T,H]; w13 [E,2F,H] (gate rows then up rows); w2 [E,H,F]; topk_w fp32 [T,k]; topk_idx [T,k].

    y[t] = Σ_j topk_w[t,j] · W2[e]·swiglu(W13[e]·x[t]),  e = topk_idx[t,j].
    """
    T, H = x.shape
    E = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    idx = topk_idx.long()
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok], w13[e])
        h = swiglu(h)
        y = F.linear(h, w2[e]).float()
        out.index_add_(0, tok, y * topk_w[tok, slot].float()[:, None])
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------------
# log-prob / entropy of the taken token from hidden states (LM head never materialised in full)
# --------------------------------------------------------------------------------------------

def logprob_entropy(hidden, lm_head_w, targets, temperature: float = 1.0, chunk: int = 4096,
                    with_entropy: bool = True):
    """Returns (logp [T] fp32, entropy [T] fp32) with logits = hidden·Wᵀ / temperature in fp32."""
    T = hidden.shape[0]
    if T == 0:
        # an empty micro-batch (a rank padded to its peers' count) still has to reach every parameter in backward
        z = hidden.float().sum(-1) + lm_head_w.float().sum() * 0.0
        return z, (z.clone() if with_entropy else None)
    lp = torch.empty(T, dtype=torch.float32, device=hidden.device)
    ent = torch.empty(T, dtype=torch.float32, device=hidden.device)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        logits = F.linear(hidden[s:e], lm_head_w).float()
        if temperature != 1.0:
            logits = logits / temperature
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(1, targets[s:e].long()[:, None]).squeeze(1)
        lp[s:e] = tgt - lse
        if with_entropy:
            p = torch.softmax(logits, dim=-1)
            ent[s:e] = lse - (p * logits).sum(-1)
    return lp, (ent if with_entropy else None)


# --------------------------------------------------------------------------------------------
# optimizer
# --------------------------------------------------------------------------------------------

def adamw_step(master, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale: float = 1.0, param_out: torch.Tensor | None = None):
    """In-place AdamW on fp32 master/moments from a (possibly bf16) gradient; optional bf16 copy-out."""
    g = grad.float() * grad_scale
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    master.mul_(1 - lr * weight_decay).addcdiv_(exp_avg / bc1, denom, value=-lr)
    if param_out is not None:
        param_out.copy_(master)


# --------------------------------------------------------------------------------------------
# quantisation
# --------------------------------------------------------------------------------------------
FP8_E4M3_MAX = 448.0
FP4_E2M1_MAX = 6.0
_E2M1_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _e8m0_from_amax(amax: torch.Tensor, elem_max: float) -> torch.Tensor:
    """Power-of-two scale exponent (biased, uint8) so that amax / 2^e ≤ elem_max: ceil(log2(amax/max))."""
    ratio = (amax.float() / elem_max).clamp_min(2.0 ** -127)
    e = torch.ceil(torch.log2(ratio)).clamp(-127, 127)
    return (e + 127).to(torch.uint8)


def mxfp8_quant(x: torch.Tensor, block: int = 32):
    """1×32 block-scaled FP8 e4m3 with e8m0 scales along the last dim.

    Returns (q float8_e4m3fn [.., N], scales uint8 [.., N/32]).
    """
    shp = x.shape
    xb = x.float().reshape(*shp[:-1], shp[-1] // block, block)
    amax = xb.abs().amax(-1)
    e = _e8m0_from_amax(amax, FP8_E4M3_MAX)
    scale = torch.exp2(e.float() - 127)
    q = (xb / scale[..., None]).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shp), e


def mxfp8_dequant(q: torch.Tensor, e: torch.Tensor, block: int = 32, dtype=torch.float32):
    shp = q.shape
    qb = q.float().reshape(*shp[:-1], shp[-1] // block, block)
    return (qb * torch.exp2(e.float() - 127)[..., None]).reshape(shp).to(dtype)


def fp8_blockwise_quant(w: torch.Tensor, block_m: int = 128, block_n: int = 128):
    """128×128-block FP8 e4m3 cast with fp32 `scale_inv` (dequant multiplier) per block."""
    M, N = w.shape
    pm, pn = (-M) % block_m, (-N) % block_n
    wf = F.pad(w.float(), (0, pn, 0, pm))
    Mb, Nb = wf.shape[0] // block_m, wf.shape[1] // block_n
    blk = wf.reshape(Mb, block_m, Nb, block_n)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale_inv = amax / FP8_E4M3_MAX
    q = (blk / scale_inv[:, None, :, None]).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    q = q.reshape(Mb * block_m, Nb * block_n)[:M, :N].to(torch.float8_e4m3fn)
    return q, scale_inv


def fp8_blockwise_dequant(q, scale_inv, block_m: int = 128, block_n: int = 128, dtype=torch.bfloat16):
    M, N = q.shape
    s = scale_inv.repeat_interleave(block_m, 0)[:M].repeat_interleave(block_n, 1)[:, :N]
    return (q.float() * s).to(dtype)


def int4_fake_quant(x: torch.Tensor, block_m: int = 1, block_n: int = 32, symmetric: bool = True):
    """Quantise→dequantise to INT4 per [block_m, block_n] block (sym: /7 ; asym: /15 with zero point)."""
    M, N = x.shape
    xb = x.float().reshape(M // block_m, block_m, N // block_n, block_n)
    if symmetric:
        amax = xb.abs().amax(dim=(1, 3), keepdim=True)
        scale = (amax / 7.0).clamp_min(1e-10)
        q = torch.round(xb / scale).clamp(-8, 7)
        out = q * scale
        scales = scale
    else:
        mx = xb.amax(dim=(1, 3), keepdim=True)
        mn = xb.amin(dim=(1, 3), keepdim=True)
        scale = ((mx - mn) / 15.0).clamp_min(1e-10)
        zp = torch.round(-mn / scale)
        q = (torch.round(xb / scale) + zp).clamp(0, 15)
        out = (q - zp) * scale
        scales = scale
    return out.reshape(M, N).to(x.dtype), scales.reshape(M // block_m, N // block_n)


def _round_e2m1(v: torch.Tensor) -> torch.Tensor:
    """Round |v| ≤ 6 to the nearest e2m1 value, ties to even mantissa (matches cvt.rn.satfinite)."""
    grid = _E2M1_GRID.to(v.device)
    a = v.abs().clamp(max=FP4_E2M1_MAX)
    idx = torch.bucketize(a, grid)  # first grid >= a
    idx = idx.clamp(1, 7)
    lo, hi = grid[idx - 1], grid[idx]
    mid = (lo + hi) / 2
    take_hi = (a > mid) | ((a == mid) & ((idx % 2) == 0))
    r = torch.where(take_hi, hi, lo)
    r = torch.where(a == 0, torch.zeros_like(r), r)
    return r * v.sign()


def nvfp4_qdq(x: torch.Tensor, global_amax: torch.Tensor | None = None, block: int = 16, four_over_six: bool = False):
    """NVFP4 quantise→dequantise: 1×16 blocks, e4m3 block scale, fp32 per-tensor scale.  `four_over_six`: per block the
    maximum is mapped to 6 or to 4, whichever gives the smaller squared error."""
    shp = x.shape
    xf = x.float().reshape(-1, block)
    gamax = x.float().abs().max() if global_amax is None else global_amax.float()
    gscale = (FP8_E4M3_MAX * FP4_E2M1_MAX) / gamax.clamp_min(1e-12)  # encode scale
    amax = xf.abs().amax(-1, keepdim=True)

    def candidate(target):
        sb = (amax / target * gscale).clamp(max=FP8_E4M3_MAX).to(torch.float8_e4m3fn).float()
        dec = sb / gscale  # decode multiplier per block
        enc = torch.where(dec > 0, 1.0 / dec, torch.zeros_like(dec))
        return _round_e2m1(xf * enc) * dec

    y = candidate(FP4_E2M1_MAX)
    if four_over_six:
        y4 = candidate(4.0)
        better = ((y4 - xf) ** 2).sum(-1, keepdim=True) < ((y - xf) ** 2).sum(-1, keepdim=True)
        y = torch.where(better, y4, y)
    return y.reshape(shp).to(x.dtype)


# --------------------------------------------------------------------------------------------
# collectives restated on one device (for fused-kernel tests): lists of per-rank tensors
# --------------------------------------------------------------------------------------------

def allreduce_add_rmsnorm(parts: list[torch.Tensor], residual: torch.Tensor, w: torch.Tensor, eps: float):
    s = torch.stack([p.float() for p in parts]).sum(0).to(parts[0].dtype)
    return add_rmsnorm(s, residual, w, eps)


# --------------------------------------------------------------------------------------------
# block fake quantisation (quantise → dequantise in the input's dtype)
# --------------------------------------------------------------------------------------------

def _ceil_pow2(v: torch.Tensor) -> torch.Tensor:
    bits = v.float().contiguous().view(torch.int32)
    e = ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return ((e + 127) << 23).view(torch.float32)


def _e2m1_round(v: torch.Tensor) -> torch.Tensor:
    mag = v.abs()
    step = torch.where(mag < 2.0, torch.full_like(mag, 0.5), torch.where(mag < 4.0, torch.ones_like(mag), torch.full_like(mag, 2.0)))
    return torch.round(mag / step) * step * torch.sign(v)          # torch.round: ties to even, like rint


def block_fake_quant(x: torch.Tensor, mode: str = "fp8") -> torch.Tensor:
    """`fp8`: 1×32 blocks, power-of-two scale, e4m3 payload (MXFP8 style).  `fp4`: the same with an e2m1 payload (MXFP4
    style).  `compressed_kv`: 1×16 blocks, e4m3 scale in [2^-9, 448], e2m1 payload.  Blocks run along the last axis.
    Reference behaviour: miles/kernels/quant/fake_quant.py:24-62."""
    block = 16 if mode == "compressed_kv" else 32
    assert x.shape[-1] % block == 0, f"last dimension must be a multiple of {block}"
    v = x.float().reshape(-1, block)
    amax = v.abs().amax(dim=1)
    if mode == "compressed_kv":
        scale = (amax * (1.0 / 6.0)).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn).float()
        fmax = 6.0
    else:
        fmax = 448.0 if mode == "fp8" else 6.0
        floor = 1e-4 if mode == "fp8" else 6 * 2.0 ** -126
        scale = _ceil_pow2(amax.clamp_min(floor) * (1.0 / fmax))
    scaled = (v / scale[:, None]).clamp(-fmax, fmax)
    q = scaled.to(torch.float8_e4m3fn).float() if mode == "fp8" else _e2m1_round(scaled)
    return (q * scale[:, None]).reshape(x.shape).to(x.dtype)
