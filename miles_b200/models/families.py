"""Model families beyond Qwen3: the layer kinds of the reference's model plugins as blocks of one configurable decoder.

The reference adds these families as Megatron layer specs plus HF↔Megatron weight bridges
(miles_plugins/models/{deepseek_v4,glm5,kimi_k3,qwen3_next,qwen3_5,…}, miles_plugins/mbridge/*.py); its rollouts for
them run on the external engine.  Here a `FamilyConfig` lists one mixer kind per layer and the decoder is assembled
from these blocks (training / scoring path: packed sequences described by `ForwardMeta.cu_seqlens`):

    full   grouped-query attention with QK-norm + RoPE (the Qwen3 block), optional sigmoid output gate and partial
           rotary dimension (Qwen3-Next / Qwen3.5 full-attention layers)
    mla    multi-head latent attention: low-rank q and kv projections, decoupled RoPE key shared by the heads
           (DeepSeek-V3 family, Kimi-K2, GLM-5)
    dsa    `mla` whose keys are picked per query by a lightning indexer (DeepSeek-V3.2 / V4 sparse attention); the
           indexer is trained with the KL of its scores against the dense attention mass (`FamilyModel.aux_losses`)
    gdn    gated delta-rule linear attention with a short causal convolution and a gated output norm (Qwen3-Next)
    kda    the delta rule with a per-channel decay gate (Kimi linear attention)

Feed-forward: dense SwiGLU, or routed experts with softmax or sigmoid(+selection bias) scores, a routed scaling factor
and always-on shared experts (DeepSeek / GLM / Kimi MoE).  `hc_streams > 1` widens the residual into that many
hyper-connection streams that every block reads through learned aggregation weights and writes through learned mixing
weights (ops.extra.mhc_*).

Tensor parallelism of the new blocks is 1 (data / expert / pipeline parallelism and ZeRO work as for Qwen3); the `full`
block and the MoE feed-forward reuse the Qwen3 modules and keep their TP / EP support.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import extra as X
from ..ops import reference as ref
from ..ops import sparse_attention as SA
from ..parallel.state import ParallelState
from .config import PRESETS, ModelConfig
from .qwen3 import Attention, DenseFFN, ForwardMeta, MoEFFN, Qwen3Model, _Init


@dataclass(frozen=True)
class FamilyConfig(ModelConfig):
    family: str = "qwen3"
    layer_types: tuple = ()                 # one of full / mla / dsa / gdn / kda per layer; () → all "full"
    # full attention extras
    attn_output_gate: bool = False
    partial_rotary: float = 1.0
    # latent attention
    q_lora_rank: int = 0
    kv_lora_rank: int = 64
    qk_nope_head_dim: int = 32
    qk_rope_head_dim: int = 16
    v_head_dim: int = 32
    # lightning indexer
    index_heads: int = 2
    index_dim: int = 32
    index_topk: int = 16
    # linear attention
    linear_heads: int = 4
    linear_key_dim: int = 32
    linear_value_dim: int = 32
    conv_kernel: int = 4
    # MoE extras
    router_score: str = "softmax"           # softmax | sigmoid
    router_bias: bool = False               # selection-only bias (aux-loss-free balancing)
    routed_scaling: float = 1.0
    n_shared_experts: int = 0
    # hyper-connections
    hc_streams: int = 1

    def layer_type(self, layer: int) -> str:
        return self.layer_types[layer] if self.layer_types else "full"


def _rms(x, w, eps):
    return ops.rmsnorm(x, w, eps)


def _seq_ids(meta: ForwardMeta, T: int, device) -> torch.Tensor:
    cu = meta.cu_seqlens.long()
    return torch.bucketize(torch.arange(T, device=device), cu[1:], right=True)


def _dense_attention(q, k, v, meta: ForwardMeta, scale: float):
    """Causal attention within each packed sequence for any head dims (q/k dim may differ from v's)."""
    D, Dv = q.shape[-1], v.shape[-1]
    if D == Dv and q.shape[1] % k.shape[1] == 0 and abs(scale - 1.0 / math.sqrt(D)) < 1e-12:
        return ops.attention_varlen(q, k, v, meta.cu_seqlens, meta.max_seqlen)
    T = q.shape[0]
    seq = _seq_ids(meta, T, q.device)
    pos = meta.positions.long()
    vis = (seq[:, None] == seq[None, :]) & (pos[None, :] <= pos[:, None])
    rep = q.shape[1] // k.shape[1]
    s = torch.einsum("thd,shd->hts", q.float(), k.float().repeat_interleave(rep, 1)) * scale
    p = torch.softmax(s.masked_fill(~vis[None], float("-inf")), -1)
    return torch.einsum("hts,shd->thd", p, v.float().repeat_interleave(rep, 1)).to(q.dtype)


class GatedAttention(Attention):
    """The Qwen3 attention block with a sigmoid gate on the attention output and rotary on a leading fraction of each head."""

    def __init__(self, cfg: FamilyConfig, ps, dtype, device, gen, tag):
        super().__init__(cfg, ps, dtype, device, gen, tag)
        assert ps.tp_size == 1
        self.w_gate = nn.Parameter(gen(f"{tag}.wgate", (cfg.q_size, cfg.hidden_size), cfg.init_std, dtype, device)) if cfg.attn_output_gate else None
        self.rot = int(cfg.head_dim * cfg.partial_rotary) // 2 * 2

    def forward(self, x, meta: ForwardMeta, layer: int, qkv=None):
        cfg, T = self.cfg, x.shape[0]
        assert meta.kv_cache is None, "this block has no paged-KV decode path"
        q, k, v = ops.linear(x, self.wqkv, self.bqkv).split([self.hq * self.d, self.hkv * self.d, self.hkv * self.d], -1)
        q, k, v = q.view(T, self.hq, self.d), k.view(T, self.hkv, self.d), v.view(T, self.hkv, self.d)
        if self.rot == self.d:
            q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, meta.positions, cfg.rope_theta, cfg.rms_eps)
        else:
            if self.q_norm is not None:
                q, k = _rms(q, self.q_norm, cfg.rms_eps), _rms(k, self.k_norm, cfg.rms_eps)
            q = torch.cat([ops.rope(q[..., :self.rot].contiguous(), meta.positions, cfg.rope_theta), q[..., self.rot:]], -1)
            k = torch.cat([ops.rope(k[..., :self.rot].contiguous(), meta.positions, cfg.rope_theta), k[..., self.rot:]], -1)
        if self.ps.cp_size > 1:
            # contiguous context-parallel chunks: swap the sequence sharding for a head sharding around the kernel (Ulysses),
            # or gather K/V (`allgather`); the recurrent layers of the same model pass their state along the same chunks
            from ..parallel import cp as _cp
            from ..parallel import cp_ring as _ring

            if self.ps.cp_comm_type == "a2a":
                qh, kh, vh = (_cp.seq_to_heads(t, self.ps) for t in (q, k, v))
                o = _cp.heads_to_seq(ops.attention_varlen(qh, kh, vh, meta.cu_seqlens, meta.max_seqlen), self.ps)
            else:
                assert self.ps.cp_comm_type == "allgather", "family models run context parallelism over contiguous chunks"
                o = _ring.allgather_attention(q, k, v, meta.cu_seqlens, self.ps)
            o = o.reshape(T, self.hq * self.d)
        else:
            o = ops.attention_varlen(q, k, v, meta.cu_seqlens, meta.max_seqlen).reshape(T, self.hq * self.d)
        if self.w_gate is not None:
            o = o * torch.sigmoid(ops.linear(x, self.w_gate))
        return ops.linear(o, self.wo)


class LatentAttention(nn.Module):
    """Multi-head latent attention; with `sparse` the keys of each query come from a lightning indexer."""

    def __init__(self, cfg: FamilyConfig, ps, dtype, device, gen, tag, sparse: bool):
        super().__init__()
        assert ps.tp_size == 1, "latent attention runs with tensor parallel size 1"
        self.cfg, self.sparse, self.ps = cfg, sparse, ps
        H, hd = cfg.hidden_size, cfg.num_heads
        self.dn, self.dr, self.dv = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        dq = self.dn + self.dr

        def P(name, shape):
            return nn.Parameter(gen(f"{tag}.{name}", shape, cfg.init_std, dtype, device))

        if cfg.q_lora_rank:
            self.wq_a, self.q_a_norm = P("wq_a", (cfg.q_lora_rank, H)), nn.Parameter(torch.ones(cfg.q_lora_rank, dtype=dtype, device=device))
            self.wq_b = P("wq_b", (hd * dq, cfg.q_lora_rank))
        else:
            self.wq = P("wq", (hd * dq, H))
        self.wkv_a = P("wkv_a", (cfg.kv_lora_rank + self.dr, H))
        self.kv_a_norm = nn.Parameter(torch.ones(cfg.kv_lora_rank, dtype=dtype, device=device))
        self.wkv_b = P("wkv_b", (hd * (self.dn + self.dv), cfg.kv_lora_rank))
        self.wo = P("wo", (H, hd * self.dv))
        if sparse:
            self.wq_idx = P("wq_idx", (cfg.index_heads * cfg.index_dim, cfg.q_lora_rank or H))
            self.wk_idx = P("wk_idx", (cfg.index_dim, H))
            self.k_idx_norm = nn.Parameter(torch.ones(cfg.index_dim, dtype=dtype, device=device))
            self.w_idx = P("w_idx", (cfg.index_heads, H))
        self.last_index_loss = None

    def forward(self, x, meta: ForwardMeta, layer: int, qkv=None):
        cfg, T, hd = self.cfg, x.shape[0], self.cfg.num_heads
        assert meta.kv_cache is None, "this block has no paged-KV decode path"
        if cfg.q_lora_rank:
            q_lat = _rms(ops.linear(x, self.wq_a), self.q_a_norm, cfg.rms_eps)
            q = ops.linear(q_lat, self.wq_b)
        else:
            q_lat, q = x, ops.linear(x, self.wq)
        q = q.view(T, hd, self.dn + self.dr)
        kv_a = ops.linear(x, self.wkv_a)
        c_kv = _rms(kv_a[:, :cfg.kv_lora_rank].contiguous(), self.kv_a_norm, cfg.rms_eps)
        k_rope = ops.rope(kv_a[:, cfg.kv_lora_rank:].reshape(T, 1, self.dr).contiguous(), meta.positions, cfg.rope_theta)
        q_rope = ops.rope(q[..., self.dn:].contiguous(), meta.positions, cfg.rope_theta)
        qf = torch.cat([q[..., :self.dn], q_rope], -1)
        scale = 1.0 / math.sqrt(self.dn + self.dr)
        self.last_index_loss = None
        if self.ps.cp_size > 1:
            idx_in = None
            if self.sparse:
                idx_in = (ops.linear(q_lat, self.wq_idx).view(T, cfg.index_heads, cfg.index_dim),
                          _rms(ops.linear(x, self.wk_idx), self.k_idx_norm, cfg.rms_eps),
                          ops.linear(x, self.w_idx).float() / math.sqrt(cfg.index_heads * cfg.index_dim))
            return ops.linear(self._attend_cp(qf, c_kv, k_rope, meta, scale, idx_in).reshape(T, hd * self.dv), self.wo)
        kv = ops.linear(c_kv, self.wkv_b).view(T, hd, self.dn + self.dv)
        kf = torch.cat([kv[..., :self.dn], k_rope.expand(T, hd, self.dr)], -1)
        v = kv[..., self.dn:]
        if not self.sparse:
            o = _dense_attention(qf, kf, v, meta, scale)
        else:
            seq = _seq_ids(meta, T, x.device)
            q_idx = ops.linear(q_lat, self.wq_idx).view(T, cfg.index_heads, cfg.index_dim)
            k_idx = _rms(ops.linear(x, self.wk_idx), self.k_idx_norm, cfg.rms_eps)
            w_idx = ops.linear(x, self.w_idx).float() / math.sqrt(cfg.index_heads * cfg.index_dim)
            pos = meta.positions.long()
            o, idx, logits = SA.dsa_attention(qf, kf, v.contiguous(), q_idx, k_idx, w_idx, min(cfg.index_topk, T), scale,
                                              None, seq, seq, pos, pos)
            if torch.is_grad_enabled():
                # train the indexer towards the attention mass of the selected keys (main branch detached)
                with torch.no_grad():
                    kg = kf.float()[idx.clamp_min(0).long()]                         # [T, K, H, D]
                    s = torch.einsum("thd,tkhd->thk", qf.float(), kg) * scale
                    s = s.masked_fill((idx < 0).unsqueeze(1), float("-inf"))
                    mass = torch.nan_to_num(torch.softmax(s, -1), nan=0.0).sum(1)    # [T, K] summed over heads
                self.last_index_loss = SA.indexer_kl_loss(logits, mass, idx)
        return ops.linear(o.reshape(T, hd * self.dv), self.wo)


def _latent_attend_cp(self, qf, c_kv, k_rope, meta: ForwardMeta, scale: float, idx_in=None):
    """Context parallelism for latent attention over contiguous chunks: what crosses ranks is the LATENT — the compressed
    key/value vector and the shared rotary key, kv_lora_rank + rope dims per token instead of heads × (nope + v) — gathered
    over the group (gradients come back with a reduce); every rank expands the gathered latents to per-head keys and values
    and its queries attend causally inside their sequences by global position."""
    from ..parallel import cp_ring as _ring

    ps, cfg, hd = self.ps, self.cfg, self.cfg.num_heads
    assert ps.cp_comm_type in ("a2a", "allgather"), "latent attention needs contiguous context-parallel chunks"
    Tl = qf.shape[0]
    total = Tl * ps.cp_size
    parts = [c_kv, k_rope.reshape(Tl, self.dr)] + ([idx_in[1]] if idx_in is not None else [])   # + the indexer's keys
    lat = torch.cat([t.to(c_kv.dtype) for t in parts], -1)
    lat = _ring._AllGatherTokens.apply(lat, ps.cp_group, ps.cp_size, ps.cp_rank)                 # [T, r + dr (+ index dim)], global order
    c_all = lat[:, :cfg.kv_lora_rank]
    kr_all = lat[:, cfg.kv_lora_rank:cfg.kv_lora_rank + self.dr].reshape(total, 1, self.dr)
    kv = ops.linear(c_all.contiguous(), self.wkv_b).view(total, hd, self.dn + self.dv)
    kf = torch.cat([kv[..., :self.dn], kr_all.expand(total, hd, self.dr)], -1)
    v = kv[..., self.dn:]
    dev = qf.device
    lo = ps.cp_rank * Tl
    q_seq, q_pos = _ring._seq_pos(torch.arange(lo, lo + Tl, device=dev), meta.cu_seqlens)
    k_seq, k_pos = _ring._seq_pos(torch.arange(total, device=dev), meta.cu_seqlens)
    if idx_in is not None:
        # indexer-selected keys: this rank's queries choose among the keys of the whole batch; the indexer's training signal
        # is this rank's share of the batch mean (gradients are summed over the group)
        q_idx, _, w_idx = idx_in
        k_idx_all = lat[:, cfg.kv_lora_rank + self.dr:]
        o, idx, logits = SA.dsa_attention(qf, kf, v.contiguous(), q_idx, k_idx_all, w_idx, min(cfg.index_topk, total), scale,
                                          None, q_seq, k_seq, q_pos, k_pos)
        if torch.is_grad_enabled():
            with torch.no_grad():
                kg = kf.float()[idx.clamp_min(0).long()]
                sc = torch.einsum("thd,tkhd->thk", qf.float(), kg) * scale
                sc = sc.masked_fill((idx < 0).unsqueeze(1), float("-inf"))
                mass = torch.nan_to_num(torch.softmax(sc, -1), nan=0.0).sum(1)
            self.last_index_loss = SA.indexer_kl_loss(logits, mass, idx) / ps.cp_size
        return o
    vis = (q_seq[:, None] == k_seq[None, :]) & (k_pos[None, :] <= q_pos[:, None])
    s = torch.einsum("thd,shd->hts", qf.float(), kf.float()) * scale
    p = torch.softmax(s.masked_fill(~vis[None], float("-inf")), -1)
    return torch.einsum("hts,shd->thd", p, v.float()).to(qf.dtype)


LatentAttention._attend_cp = _latent_attend_cp


def delta_rule(q, k, v, beta, g, cu_seqlens, S0=None, return_state: bool = False):
    """Gated delta rule over packed sequences (fp32 state, one recurrence per sequence and head):
        S ← S ⊙ exp(g_t);  S ← S + k_t ⊗ β_t (v_t − Sᵀ k_t);  o_t = Sᵀ q_t
    q, k [T, H, dk] (already normalised / scaled), v [T, H, dv], beta [T, H], g [T, H] or [T, H, dk] (log decay ≤ 0).
    `S0` [H, dk, dv]: the state the FIRST sequence starts from (a sequence that began on another context-parallel rank);
    `return_state`: also return the state after the LAST sequence's final token."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    gf = g.float().exp()
    gf = gf[..., None, None] if gf.dim() == 2 else gf[..., None]               # [T, H, 1|dk, 1]
    out = []
    cu = cu_seqlens.tolist()
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device)
    for b in range(len(cu) - 1):
        S = S0.float() if (b == 0 and S0 is not None) else torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device)
        for t in range(cu[b], cu[b + 1]):
            S = S * gf[t]
            mem = torch.einsum("hkv,hk->hv", S, kf[t])
            S = S + torch.einsum("hk,hv->hkv", kf[t], (vf[t] - mem) * bf[t, :, None])
            out.append(torch.einsum("hkv,hk->hv", S, qf[t]))
    o = torch.stack(out).to(v.dtype) if out else v.new_zeros(0, H, dv)
    return (o, S) if return_state else o


# ---- context parallelism for the recurrent mixer: the state (and the convolution's history) travels from rank to rank ----

class _RecvFrom(torch.autograd.Function):
    """Forward: receive a tensor shaped like `like` from `src`; backward: send its gradient back there."""

    @staticmethod
    def forward(ctx, like, src, group):
        import torch.distributed as dist

        ctx.src, ctx.group = src, group
        buf = torch.empty_like(like)
        dist.recv(buf, src=src, group=group)
        return buf

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        dist.send(g.contiguous(), dst=ctx.src, group=ctx.group)
        return torch.zeros_like(g), None, None


class _SendTo(torch.autograd.Function):
    """Forward: send `t` to `dst` and return a zero scalar that ties the send into the graph; backward: receive the
    gradient of what was sent."""

    @staticmethod
    def forward(ctx, t, dst, group):
        import torch.distributed as dist

        ctx.dst, ctx.group, ctx.shape, ctx.dtype = dst, group, t.shape, t.dtype
        dist.send(t.detach().contiguous(), dst=dst, group=group)
        return t.new_zeros(())

    @staticmethod
    def backward(ctx, _):
        import torch.distributed as dist

        g = torch.empty(ctx.shape, dtype=ctx.dtype, device=_.device)
        dist.recv(g, src=ctx.dst, group=ctx.group)
        return g, None, None


def local_segments(cu_seqlens, lo: int, hi: int):
    """Sequence boundaries of the packed batch inside the token range [lo, hi), relative to lo, and whether the first and the
    last local segment continue from / into a neighbouring range."""
    cu = [int(c) for c in cu_seqlens.tolist()]
    if cu[-1] < hi:
        cu.append(hi)                                    # padding tokens past the last sequence form one more segment
    inner = [c for c in cu if lo < c < hi]
    bounds = [lo] + inner + [hi]
    return [b - lo for b in bounds], lo not in cu, hi not in cu


class LinearAttention(nn.Module):
    """Gated delta-rule mixer: projections → short causal conv + SiLU on q/k/v → L2-normalised q, k → delta rule →
    per-head RMSNorm gated by silu(z) → output projection.  `per_channel_decay` gives the decay one gate per key channel
    (Kimi delta attention) instead of one per head (gated DeltaNet)."""

    def __init__(self, cfg: FamilyConfig, ps, dtype, device, gen, tag, per_channel_decay: bool):
        super().__init__()
        assert ps.tp_size == 1, "linear attention runs with tensor parallel size 1"
        self.cfg, self.per_channel, self.ps = cfg, per_channel_decay, ps
        H, nh, dk, dv = cfg.hidden_size, cfg.linear_heads, cfg.linear_key_dim, cfg.linear_value_dim
        self.nh, self.dk, self.dv = nh, dk, dv

        def P(name, shape):
            return nn.Parameter(gen(f"{tag}.{name}", shape, cfg.init_std, dtype, device))

        self.w_qkvz = P("w_qkvz", (nh * (2 * dk + 2 * dv), H))
        self.w_ba = P("w_ba", (nh * (1 + (dk if per_channel_decay else 1)), H))
        self.conv = P("conv", (nh * (2 * dk + dv), cfg.conv_kernel))
        self.A_log = nn.Parameter(torch.zeros(nh, dtype=torch.float32, device=device))
        self.dt_bias = nn.Parameter(torch.zeros(nh * (dk if per_channel_decay else 1), dtype=torch.float32, device=device))
        self.o_norm = nn.Parameter(torch.ones(dv, dtype=dtype, device=device))
        self.wo = P("wo", (H, nh * dv))

    def forward(self, x, meta: ForwardMeta, layer: int, qkv=None):
        assert meta.kv_cache is None, "this block has no recurrent-state decode path"
        cfg, T, nh, dk, dv = self.cfg, x.shape[0], self.nh, self.dk, self.dv
        qkvz = ops.linear(x, self.w_qkvz)
        qkv_, z = qkvz[:, :nh * (2 * dk + dv)], qkvz[:, nh * (2 * dk + dv):].reshape(T, nh, dv)
        if self.ps.cp_size > 1:
            return self._forward_cp(x, meta, qkv_, z)
        seqlens = (meta.cu_seqlens[1:] - meta.cu_seqlens[:-1]).to(torch.int32)
        qkv_ = F.silu(X.short_conv_fp32(qkv_.contiguous(), self.conv, seqlens).float())
        o = self._mix(x, qkv_, meta.cu_seqlens)
        return self._finish(x, o, z)

    def _mix(self, x, qkv_, cu_seqlens, S0=None, return_state: bool = False):
        T, nh, dk, dv = x.shape[0], self.nh, self.dk, self.dv
        q, k, v = qkv_.split([nh * dk, nh * dk, nh * dv], -1)
        q = F.normalize(q.reshape(T, nh, dk), dim=-1) / math.sqrt(dk)
        k = F.normalize(k.reshape(T, nh, dk), dim=-1)
        ba = ops.linear(x, self.w_ba).float()
        beta = torch.sigmoid(ba[:, :nh])
        a = ba[:, nh:] + self.dt_bias
        g = -torch.exp(self.A_log)[None, :, None] * F.softplus(a.reshape(T, nh, -1))          # log decay ≤ 0
        g = g if self.per_channel else g.squeeze(-1)
        return delta_rule(q, k, v.reshape(T, nh, dv), beta, g, cu_seqlens, S0=S0, return_state=return_state)

    def _finish(self, x, o, z):
        cfg, T = self.cfg, x.shape[0]
        o = _rms(o.to(x.dtype), self.o_norm, cfg.rms_eps) * F.silu(z.float()).to(x.dtype)
        return ops.linear(o.reshape(T, self.nh * self.dv), self.wo)

    def _forward_cp(self, x, meta, qkv_, z):
        """Context parallelism with contiguous token chunks (the layout of `--cp-comm-type a2a` / `allgather`): a sequence
        cut by a chunk boundary continues on the next rank from the state this rank ends with, and its convolution sees this
        rank's last W − 1 inputs.  Both travel in ONE message per boundary (and their gradients in one message back), ranks
        compute their chunks one after another along each cut sequence.  The reference does this for its linear-attention
        families through fla's state passing (miles_plugins/models/hf_attention.py:184-199)."""
        from ..parallel.cp import chunk_bounds

        ps = self.ps
        assert ps.cp_comm_type in ("a2a", "allgather"), "the recurrent mixer needs contiguous context-parallel chunks"
        T, nh, dk, dv, W = x.shape[0], self.nh, self.dk, self.dv, self.conv.shape[1]
        lo, hi = chunk_bounds(T * ps.cp_size, ps.cp_size, ps.cp_rank)
        bounds, from_prev, to_next = local_segments(meta.cu_seqlens, lo, hi)
        C = qkv_.shape[1]
        n_state, n_halo = nh * dk * dv, (W - 1) * C
        pre = qkv_.float()
        S0, halo = None, None
        if from_prev and ps.cp_rank > 0:
            like = torch.zeros(n_state + n_halo, dtype=torch.float32, device=x.device, requires_grad=torch.is_grad_enabled())
            msg = _RecvFrom.apply(like, ps.cp_ranks[ps.cp_rank - 1], ps.cp_group)
            S0, halo = msg[:n_state].view(nh, dk, dv), msg[n_state:].view(W - 1, C)
        # causal convolution: the first segment is extended by the neighbour's last W − 1 inputs (zeros where that sequence is shorter)
        ext = torch.cat([halo, pre]) if halo is not None else pre
        shift = (W - 1) if halo is not None else 0
        seg = [b + shift for b in bounds]
        seg[0] = 0
        seqlens = torch.tensor([b - a for a, b in zip(seg[:-1], seg[1:])], dtype=torch.int32, device=x.device)
        conv = X.short_conv_fp32(ext.contiguous(), self.conv, seqlens).float()[shift:]
        cu_local = torch.tensor(bounds, dtype=torch.int32, device=x.device)
        o, S_last = self._mix(x, F.silu(conv), cu_local, S0=S0, return_state=True)
        out = self._finish(x, o, z)
        if to_next and ps.cp_rank < ps.cp_size - 1:
            first_of_last = seg[-2]                                     # the cut sequence's rows in `ext` (halo rows included)
            tail = ext[max(first_of_last, ext.shape[0] - (W - 1)):]
            tail = torch.cat([tail.new_zeros(W - 1 - tail.shape[0], C), tail]) if tail.shape[0] < W - 1 else tail
            tie = _SendTo.apply(torch.cat([S_last.reshape(-1), tail.reshape(-1)]), ps.cp_ranks[ps.cp_rank + 1], ps.cp_group)
            out = out + tie.to(out.dtype)
        return out

        o = _rms(o.to(x.dtype), self.o_norm, cfg.rms_eps) * F.silu(z.float()).to(x.dtype)
        return ops.linear(o.reshape(T, nh * dv), self.wo)


class FamilyMoE(MoEFFN):
    """Routed experts with softmax or sigmoid scores, a selection-only bias, a routed scaling factor and shared experts."""

    def __init__(self, cfg: FamilyConfig, ps, dtype, device, gen, tag, moe_index: int):
        super().__init__(cfg, ps, dtype, device, gen, tag, moe_index)
        self.e_bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=torch.float32, device=device), requires_grad=False) if cfg.router_bias else None
        self.shared = None
        if cfg.n_shared_experts:
            shared_cfg = cfg.with_(ffn_hidden_size=cfg.moe_ffn_hidden_size * cfg.n_shared_experts)
            self.shared = DenseFFN(shared_cfg, ps, dtype, device, gen, f"{tag}.shared")

    def forward(self, x, meta: ForwardMeta, layer: int, logits=None):
        cfg = self.cfg
        logits = ops.linear_fp32(x, self.router)
        k = cfg.moe_topk
        if cfg.router_score == "sigmoid":
            scores = torch.sigmoid(logits)
            pick = scores + self.e_bias if self.e_bias is not None else scores
        else:
            scores = torch.softmax(logits, -1)
            pick = scores
        if meta.replay_topk is not None:
            idx = self.ps.sp_slice(meta.replay_topk)[:, self.moe_index, :].long()
            bad = (idx < 0).all(-1, keepdim=True)
            idx = torch.where(bad, pick.topk(k, -1).indices, idx.clamp_min(0))
        else:
            idx = pick.topk(k, -1).indices
        w = scores.gather(-1, idx)
        if cfg.moe_norm_topk_prob:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        w = w * cfg.routed_scaling
        if meta.record_topk is not None:
            meta.record_topk.append(idx.to(torch.int32).detach())
        y = self.ps.moe_ffn(x, self.w13, self.w2, w, idx.to(torch.int32), cfg.num_experts)
        return y + self.shared(x, meta, layer) if self.shared is not None else y


class FamilyLayer(nn.Module):
    def __init__(self, cfg: FamilyConfig, ps, dtype, device, gen, layer: int, moe_index: int):
        super().__init__()
        self.layer, self.eps, self.n = layer, cfg.rms_eps, cfg.hc_streams
        tag, kind = f"L{layer}", cfg.layer_type(layer)
        self.ln1 = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.ln2 = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        if kind == "full":
            plain = not cfg.attn_output_gate and cfg.partial_rotary == 1.0
            self.attn = Attention(cfg, ps, dtype, device, gen, tag) if plain else GatedAttention(cfg, ps, dtype, device, gen, tag)
        elif kind in ("mla", "dsa"):
            self.attn = LatentAttention(cfg, ps, dtype, device, gen, tag, sparse=kind == "dsa")
        elif kind in ("gdn", "kda"):
            self.attn = LinearAttention(cfg, ps, dtype, device, gen, tag, per_channel_decay=kind == "kda")
        else:
            raise ValueError(f"unknown layer type '{kind}'")
        if cfg.layer_is_moe(layer):
            special = cfg.router_score != "softmax" or cfg.router_bias or cfg.n_shared_experts or cfg.routed_scaling != 1.0
            self.mlp = (FamilyMoE if special else MoEFFN)(cfg, ps, dtype, device, gen, tag, moe_index)
        else:
            self.mlp = DenseFFN(cfg, ps, dtype, device, gen, tag)
        if self.n > 1:
            # per block: read weights over the streams, write weights, and a stream-mixing matrix (identity at init)
            n = self.n
            self.hc = nn.ParameterDict({
                f"{b}_{w}": nn.Parameter(v.to(torch.float32).to(device))
                for b in ("attn", "mlp")
                for w, v in (("pre", torch.full((n,), 1.0 / n)), ("post", torch.ones(n)), ("res", torch.eye(n)))})

    def _block(self, streams, fn, norm_w, name, meta):
        n = self.n
        pre, post, res = self.hc[f"{name}_pre"], self.hc[f"{name}_post"], self.hc[f"{name}_res"]
        x = X.mhc_aggregate(streams, pre, n).to(streams.dtype)
        y = fn(_rms(x, norm_w, self.eps), meta, self.layer)
        return X.mhc_mix(y, streams, res, post, n)

    def forward(self, x, residual, meta: ForwardMeta):
        if self.n > 1:
            # `x` carries the n streams side by side ([T, n·H]); no separate residual
            x = self._block(x, self.attn, self.ln1, "attn", meta)
            x = self._block(x, self.mlp, self.ln2, "mlp", meta)
            return x, None
        h, residual = ops.add_rmsnorm(x, residual, self.ln1, self.eps)
        h = self.attn(h, meta, self.layer)
        h, residual = ops.add_rmsnorm(h, residual, self.ln2, self.eps)
        return self.mlp(h, meta, self.layer), residual


class FamilyModel(Qwen3Model):
    """Decoder assembled from `FamilyConfig.layer_types`; same interface as `Qwen3Model` for the trainer."""

    def __init__(self, cfg: FamilyConfig, ps: ParallelState | None = None, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                 layer_range=None):
        super().__init__(cfg.with_(num_layers=0), ps, dtype=dtype, device=device, seed=seed, layer_range=(0, 0))
        self.cfg = cfg
        gen = _Init(seed)
        lo, hi = layer_range or (0, cfg.num_layers)
        assert (lo, hi) == (0, cfg.num_layers) or cfg.hc_streams == 1, "hyper-connection streams do not cross pipeline stages"
        self.layer_range, self.has_embed, self.has_head = (lo, hi), lo == 0, hi == cfg.num_layers
        layers, moe_index = [], 0
        for l in range(cfg.num_layers):
            if lo <= l < hi:
                layers.append(FamilyLayer(cfg, self.ps, dtype, device, gen, l, moe_index))
            moe_index += int(cfg.layer_is_moe(l))
        self.layers = nn.ModuleList(layers)
        self.num_moe_layers = moe_index
        # only the plain Qwen3 attention block has a paged-KV decode path; engines serve the others by re-scoring
        self.supports_kv_cache = all(type(l.attn) is Attention for l in layers)
        if not self.has_embed:
            self.embed = None
        if not self.has_head:
            self.norm = self.lm_head = None

    def forward(self, tokens, meta: ForwardMeta, hidden_in=None):
        n = self.cfg.hc_streams
        x = ops.embedding(tokens, self.embed) if self.has_embed else hidden_in
        if n > 1 and self.has_embed:
            x = x.repeat(1, n)
        residual = None
        for layer in self.layers:
            x, residual = layer(x, residual, meta)
        if not self.has_head:
            return x if residual is None else x + residual
        if n > 1:
            x = x.view(x.shape[0], n, -1).float().sum(1).to(x.dtype)
        h, _ = ops.add_rmsnorm(x, residual, self.norm, self.cfg.rms_eps)
        return h

    def aux_losses(self) -> dict:
        """Auxiliary training losses of the last forward (the sparse-attention indexer's KL), to be added to the objective."""
        terms = [l.attn.last_index_loss for l in self.layers if getattr(l.attn, "last_index_loss", None) is not None]
        return {"indexer_kl": torch.stack(terms).mean()} if terms else {}

    @torch.no_grad()
    def update_router_bias(self, counts_per_layer: list, rate: float = 1e-3):
        """Aux-loss-free balancing: raise the selection bias of under-used experts and lower it for over-used ones.
        counts_per_layer: one [num_experts] token-count tensor per MoE layer (e.g. from recorded routing)."""
        moes = [l.mlp for l in self.layers if isinstance(l.mlp, FamilyMoE) and l.mlp.e_bias is not None]
        for m, c in zip(moes, counts_per_layer):
            c = c.float().to(m.e_bias.device)
            m.e_bias.add_(rate * torch.sign(c.mean() - c))


def provider(cfg, ps, dtype, device, seed=0):
    """`--custom-model-provider-path miles_b200.models.families:provider`."""
    return build_family_model(cfg, ps, dtype=dtype, device=device, seed=seed)


def build_family_model(cfg: FamilyConfig, ps=None, dtype=torch.bfloat16, device="cpu", seed: int = 0):
    ps = ps or ParallelState.single()
    layer_range = None
    if ps.pp_size > 1:
        per = math.ceil(cfg.num_layers / ps.pp_size)
        layer_range = (ps.pp_rank * per, min(cfg.num_layers, (ps.pp_rank + 1) * per))
    return FamilyModel(cfg, ps, dtype=dtype, device=device, seed=seed, layer_range=layer_range)


_T = dict(vocab_size=512, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, ffn_hidden_size=256)

FAMILY_PRESETS: dict[str, FamilyConfig] = {
    # DeepSeek-V3.2 / V4 shape: latent attention everywhere, indexer-selected keys, sigmoid router with bias, shared expert
    "deepseek-tiny": FamilyConfig(name="deepseek-tiny", family="deepseek_v32", num_layers=3, layer_types=("mla", "dsa", "dsa"),
                                  q_lora_rank=48, num_experts=8, moe_topk=2, moe_ffn_hidden_size=64, first_k_dense=1,
                                  router_score="sigmoid", router_bias=True, routed_scaling=2.5, n_shared_experts=1, **_T),
    # GLM-4.5/5 shape: grouped-query attention with partial rotary, sigmoid-routed MoE with a shared expert after a dense layer
    "glm-moe-tiny": FamilyConfig(name="glm-moe-tiny", family="glm4_moe", num_layers=2, partial_rotary=0.5, num_experts=8,
                                 moe_topk=2, moe_ffn_hidden_size=64, first_k_dense=1, router_score="sigmoid", router_bias=True,
                                 n_shared_experts=1, **_T),
    # Qwen3-Next / Qwen3.5 shape: three gated-DeltaNet layers per gated full-attention layer
    "qwen3-next-tiny": FamilyConfig(name="qwen3-next-tiny", family="qwen3_next", num_layers=4,
                                    layer_types=("gdn", "gdn", "gdn", "full"), attn_output_gate=True, partial_rotary=0.25,
                                    num_experts=8, moe_topk=2, moe_ffn_hidden_size=64, n_shared_experts=1, **_T),
    # Kimi linear shape: channel-wise delta attention interleaved with latent attention
    "kimi-linear-tiny": FamilyConfig(name="kimi-linear-tiny", family="kimi_linear", num_layers=4,
                                     layer_types=("kda", "kda", "kda", "mla"), num_experts=8, moe_topk=2,
                                     moe_ffn_hidden_size=64, first_k_dense=1, router_score="sigmoid", n_shared_experts=1, **_T),
    # hyper-connected residual streams (DeepSeek-V4 / mHC) over the plain block
    "hyper-tiny": FamilyConfig(name="hyper-tiny", family="hyper", num_layers=2, hc_streams=4, **_T),
}
PRESETS.update(FAMILY_PRESETS)
