"""Qwen2/Qwen3 dense and Qwen3-MoE decoder.

One implementation serves the trainer (packed THD forward + autograd) and the rollout engine
(paged-KV prefill/decode) so that both sides run the same kernels in the same reduction order —
the reference needs a separate "true on-policy" subsystem to approach that
(miles/true_on_policy/*); here it is structural.

Parameter layout (our own, chosen for the kernels):
  embed [V,H] · per layer: ln1 [H], wqkv [(Hq+2Hkv)·D, H] (q rows, k rows, v rows), q_norm/k_norm [D],
  wo [H, Hq·D], ln2 [H], dense FFN w13 [2F,H] (gate rows, up rows) + w2 [H,F], or MoE router [E,H],
  experts w13 [E_local,2F,H], w2 [E_local,H,F] · norm [H] · lm_head [V,H].
HF names are produced by `miles_b200.models.convert`; tensor/expert parallel shards are slices of
these tensors along dim 0 (column) or dim 1 (row).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.nn as nn

from .. import ops
from ..parallel.state import ParallelState
from .config import ModelConfig


@dataclass
class ForwardMeta:
    """Per-call description of the packed token batch."""

    positions: torch.Tensor                  # int32 [T]
    cu_seqlens: torch.Tensor | None = None   # int32 [B+1] (training / prefill without cache)
    max_seqlen: int = 0
    # paged-KV (engine) fields
    kv_cache: "list[tuple[torch.Tensor, torch.Tensor]] | None" = None
    block_table: torch.Tensor | None = None  # int32 [B, max_blocks]
    seq_lens: torch.Tensor | None = None     # int32 [B], KV length including new tokens
    q_lens: torch.Tensor | None = None       # int32 [B] new tokens per request (None → decode, 1 each)
    slot_mapping: torch.Tensor | None = None  # int64 [T] flat cache slot for each new token
    # routing replay / recording
    replay_topk: torch.Tensor | None = None  # int32 [T, L_moe, k] recorded indices (-1 rows → fallthrough)
    record_topk: "list[torch.Tensor] | None" = None  # filled with int32 [T,k] per MoE layer when not None
    recompute: bool = False                  # activation checkpoint each layer
    lora_slots: torch.Tensor | None = None   # int64 [T] adapter slot per token (None → slot 0; -1 → base model only)
    # prefill that continues cached KV (a prefix-cache hit, a later piece of a chunked prompt): packed offsets of the new
    # tokens (cu_q) and of every request's keys (cu_k), flat cache slots of those keys (kv_slots), longest key sequence (max_k)
    extend: "dict | None" = None


class _Init:
    """Deterministic N(0, std) draws keyed by a tag, independent of the parallel layout.

    Small tensors are drawn on the CPU (bit-identical on every machine, used by the tests);
    tensors on a CUDA device are drawn on that device so a 30B-parameter random init takes seconds.
    """

    def __init__(self, seed: int):
        self.seed = seed

    def __call__(self, tag: str, shape, std, dtype, device):
        import zlib

        s = (self.seed * 1000003 + zlib.crc32(tag.encode())) % (2 ** 31)
        dev = torch.device(device)
        if dev.type == "cuda":
            g = torch.Generator(device=dev).manual_seed(s)
            t = torch.empty(shape, dtype=torch.float32, device=dev)
            t.normal_(0.0, std, generator=g)
            return t.to(dtype)
        g = torch.Generator(device="cpu").manual_seed(s)
        t = torch.empty(shape, dtype=torch.float32)
        t.normal_(0.0, std, generator=g)
        return t.to(dtype)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype, device, gen, tag):
        super().__init__()
        self.cfg, self.ps = cfg, ps
        tp = ps.tp_size
        assert cfg.num_heads % tp == 0 and cfg.num_kv_heads % tp == 0, "heads must divide tp"
        self.hq, self.hkv, self.d = cfg.num_heads // tp, cfg.num_kv_heads // tp, cfg.head_dim
        full = gen(f"{tag}.wqkv", (cfg.qkv_size, cfg.hidden_size), cfg.init_std, dtype, device)
        self.wqkv = nn.Parameter(shard_qkv(full, cfg, ps.tp_rank, tp))
        self.bqkv = None
        if cfg.qkv_bias:
            self.bqkv = nn.Parameter(torch.zeros(self.wqkv.shape[0], dtype=dtype, device=device))
        wo = gen(f"{tag}.wo", (cfg.hidden_size, cfg.q_size), cfg.init_std, dtype, device)
        self.wo = nn.Parameter(wo.chunk(tp, dim=1)[ps.tp_rank].contiguous())
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
        else:
            self.q_norm = self.k_norm = None

    def forward(self, x: torch.Tensor, meta: ForwardMeta, layer: int, qkv: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        lora = getattr(self, "lora", None)
        if qkv is None:                                                   # else: computed by the caller's fused norm + projection
            qkv = self.ps.column_linear(x, self.wqkv, self.bqkv)          # SP all-gather fused on GPU
            if lora is not None and "wqkv" in lora:
                qkv = qkv + lora["wqkv"](x, meta)
        T = qkv.shape[0]
        q, k, v = qkv.split([self.hq * self.d, self.hkv * self.d, self.hkv * self.d], dim=-1)
        q, k, v = q.view(T, self.hq, self.d), k.view(T, self.hkv, self.d), v.view(T, self.hkv, self.d)
        if meta.kv_cache is not None:
            kc, vc = meta.kv_cache[layer]
            q, k = ops.qk_norm_rope_cache(q, k, v, self.q_norm, self.k_norm, meta.positions, cfg.rope_theta, cfg.rms_eps,
                                          kc, vc, meta.slot_mapping)
        else:
            q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, meta.positions, cfg.rope_theta, cfg.rms_eps)
        if meta.cu_seqlens is not None:
            # training, or an engine prefill that starts from an empty cache: attend within the new tokens
            if self.ps.cp_size > 1 and not self.ps.is_ulysses_cp:
                # ring (zigzag pieces, K/V travel round the group) or all-gather context parallelism
                from ..parallel import cp_ring as _ring
                fn = {"allgather": _ring.allgather_attention, "a2a+p2p": _ring.hierarchical_attention}.get(
                    self.ps.cp_comm_type, _ring.ring_attention)
                o = fn(q, k, v, meta.cu_seqlens, self.ps)
            elif self.ps.cp_size > 1:
                # context parallel (Ulysses): tokens are sharded in contiguous chunks; swap to a head sharding for the
                # kernel (cu_seqlens describe the whole packed batch) and back
                from ..parallel import cp as _cp
                q, k, v = (_cp.seq_to_heads(t, self.ps) for t in (q, k, v))
                o = _cp.heads_to_seq(ops.attention_varlen(q, k, v, meta.cu_seqlens, meta.max_seqlen), self.ps)
            else:
                o = ops.attention_varlen(q, k, v, meta.cu_seqlens, meta.max_seqlen)
        else:
            kc, vc = meta.kv_cache[layer]
            o = ops.paged_attention(q, kc, vc, meta.block_table, meta.seq_lens, q_lens=meta.q_lens,
                                    max_q_len=meta.max_seqlen, extend=meta.extend)
        o = o.reshape(T, self.hq * self.d)
        if lora is None and self.ps.defer_allreduce(o):
            return self.ps.row_linear_partial(o, self.wo)             # reduced inside the next add + RMSNorm kernel
        out = self.ps.row_linear(o, self.wo)                          # reduce-scatter fused on GPU
        if lora is not None and "wo" in lora:
            out = out + lora["wo"](o, meta)
        return out


class DenseFFN(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype, device, gen, tag):
        super().__init__()
        self.ps = ps
        tp, F = ps.tp_size, cfg.ffn_hidden_size
        w13 = gen(f"{tag}.w13", (2 * F, cfg.hidden_size), cfg.init_std, dtype, device)
        g, u = w13.chunk(2, dim=0)
        self.w13 = nn.Parameter(torch.cat([g.chunk(tp, 0)[ps.tp_rank], u.chunk(tp, 0)[ps.tp_rank]], 0).contiguous())
        w2 = gen(f"{tag}.w2", (cfg.hidden_size, F), cfg.init_std, dtype, device)
        self.w2 = nn.Parameter(w2.chunk(tp, dim=1)[ps.tp_rank].contiguous())

    def forward(self, x, meta: ForwardMeta, layer: int):
        lora = getattr(self, "lora", None)
        h13 = self.ps.column_linear(x, self.w13)
        if lora is not None and "w13" in lora:
            h13 = h13 + lora["w13"](x, meta)
        h = ops.swiglu(h13)
        if lora is None and self.ps.defer_allreduce(h):
            return self.ps.row_linear_partial(h, self.w2)             # reduced inside the next add + RMSNorm kernel
        out = self.ps.row_linear(h, self.w2)
        if lora is not None and "w2" in lora:
            out = out + lora["w2"](h, meta)
        return out


class MoEFFN(nn.Module):
    """Softmax top-k routed experts; experts sharded over the EP group (contiguous expert ranges)."""

    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype, device, gen, tag, moe_index: int):
        super().__init__()
        self.cfg, self.ps, self.moe_index = cfg, ps, moe_index
        E, F, H = cfg.num_experts, cfg.moe_ffn_hidden_size, cfg.hidden_size
        assert E % ps.ep_size == 0
        self.e_local = E // ps.ep_size
        self.router = nn.Parameter(gen(f"{tag}.router", (E, H), cfg.init_std, dtype, device))
        lo = ps.ep_rank * self.e_local
        # one draw per global expert id, so any EP layout starts from the same weights
        w13 = torch.empty(self.e_local, 2 * F, H, dtype=dtype, device=device)
        w2 = torch.empty(self.e_local, H, F, dtype=dtype, device=device)
        for e in range(lo, lo + self.e_local):
            w13[e - lo].copy_(gen(f"{tag}.e{e}.w13", (2 * F, H), cfg.init_std, dtype, device))
            w2[e - lo].copy_(gen(f"{tag}.e{e}.w2", (H, F), cfg.init_std, dtype, device))
        self.w13, self.w2 = nn.Parameter(w13), nn.Parameter(w2)

    def forward(self, x, meta: ForwardMeta, layer: int, logits: torch.Tensor | None = None):
        # with sequence parallelism each TP rank routes its own token slice (expert-TP is 1)
        if logits is None:
            logits = ops.linear_fp32(x, self.router)  # router scores stay fp32 (no bf16 rounding, no cast kernel)
        k, norm = self.cfg.moe_topk, self.cfg.moe_norm_topk_prob
        if meta.replay_topk is not None:
            # R3: recorded indices replace top-k, weights come from the current scores so the gate
            # still receives gradient (reference: miles/utils/replay_base.py:87-144).
            probs = torch.softmax(logits, dim=-1)
            idx = self.ps.sp_slice(meta.replay_topk)[:, self.moe_index, :]
            bad = (idx < 0).all(dim=-1)
            if bad.any():
                _, fresh, _ = ops.router_topk(logits, k, norm)
                idx = torch.where(bad[:, None], fresh, idx)
            w = ops.gather_router_weights(probs, idx, norm)
        else:
            w, idx, _ = ops.router_topk(logits, k, norm)
        if meta.record_topk is not None:
            meta.record_topk.append(idx.detach())
        return self.ps.moe_ffn(x, self.w13, self.w2, w, idx, self.cfg.num_experts)


def add_rmsnorm_reducing(ps, x, residual, w, eps):
    """add + RMSNorm; when `x` is a tensor-parallel partial sum (see `ParallelState.defer_allreduce`) the all-reduce over
    the TP ranks happens inside the same kernel, reading the peers' partial rows over NVLink."""
    if getattr(x, "_tp_partial", False):
        return ps.allreduce_add_rmsnorm(x, residual, w, eps)
    return ops.add_rmsnorm(x, residual, w, eps)


class DecoderLayer(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen, layer: int, moe_index: int):
        super().__init__()
        self.layer = layer
        self.eps = cfg.rms_eps
        self.ln1 = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        tag = f"L{layer}"
        self.attn = Attention(cfg, ps, dtype, device, gen, tag)
        self.ln2 = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.mlp = (MoEFFN(cfg, ps, dtype, device, gen, tag, moe_index) if cfg.layer_is_moe(layer)
                    else DenseFFN(cfg, ps, dtype, device, gen, tag))

    def _forward_few_tokens(self, x, residual, meta: ForwardMeta):
        """Decode with a handful of rows: each norm is fused into the matrix-vector projection that consumes it."""
        attn, mlp = self.attn, self.mlp
        qkv, residual, _ = ops.add_rmsnorm_linear(x, residual, self.ln1, self.eps, attn.wqkv, attn.bqkv)
        h = attn(None, meta, self.layer, qkv=qkv)
        if isinstance(mlp, MoEFFN):
            logits, residual, hn = ops.add_rmsnorm_linear(h, residual, self.ln2, self.eps, mlp.router, want_normed=True,
                                                          out_fp32=True)
            return mlp(hn, meta, self.layer, logits=logits), residual
        h13, residual, _ = ops.add_rmsnorm_linear(h, residual, self.ln2, self.eps, mlp.w13)
        return ops.linear(ops.swiglu(h13), mlp.w2), residual

    def forward(self, x, residual, meta: ForwardMeta):
        # `x` is the previous block's output still to be added to `residual`
        if (self.attn.ps.tp_size == 1 and ops.few_token_decode(x, self.attn.wqkv) and getattr(self.attn, "lora", None) is None
                and getattr(self.mlp, "lora", None) is None):
            return self._forward_few_tokens(x, residual, meta)
        h, residual = add_rmsnorm_reducing(self.attn.ps, x, residual, self.ln1, self.eps)
        h = self.attn(h, meta, self.layer)
        h, residual = add_rmsnorm_reducing(self.attn.ps, h, residual, self.ln2, self.eps)
        h = self.mlp(h, meta, self.layer)
        return h, residual


class Qwen3Model(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState | None = None, dtype=torch.bfloat16,
                 device="cpu", seed: int = 0, layer_range: tuple[int, int] | None = None):
        super().__init__()
        self.cfg = cfg
        self.ps = ps or ParallelState.single()
        self.dtype = dtype
        gen = _Init(seed)
        lo, hi = layer_range or (0, cfg.num_layers)
        self.layer_range = (lo, hi)
        self.has_embed = lo == 0
        self.has_head = hi == cfg.num_layers
        self.embed = (nn.Parameter(gen("embed", (cfg.vocab_size, cfg.hidden_size), cfg.init_std, dtype, device))
                      if self.has_embed else None)
        layers, moe_index = [], 0
        for l in range(cfg.num_layers):
            if lo <= l < hi:
                layers.append(DecoderLayer(cfg, self.ps, dtype, device, gen, l, moe_index))
            moe_index += int(cfg.layer_is_moe(l))
        self.layers = nn.ModuleList(layers)
        self.num_moe_layers = moe_index
        if self.has_head:
            self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
            if cfg.tie_embeddings and self.has_embed:
                self.lm_head = None
            else:
                full = gen("lm_head", (cfg.vocab_size, cfg.hidden_size), cfg.init_std, dtype, device)
                tp = self.ps.tp_size
                self.lm_head = nn.Parameter(full.chunk(tp, 0)[self.ps.tp_rank].contiguous() if tp > 1 else full)

    # ---- helpers -------------------------------------------------------------------------
    def head_weight(self) -> torch.Tensor:
        if self.lm_head is not None:
            return self.lm_head
        tp = self.ps.tp_size
        return self.embed if tp == 1 else self.embed.chunk(tp, 0)[self.ps.tp_rank]

    def forward(self, tokens: torch.Tensor, meta: ForwardMeta, hidden_in: torch.Tensor | None = None,
                inputs_embeds: torch.Tensor | None = None):
        """tokens int [T] → final-norm hidden states [T(/tp with SP), H] (last stage) or raw hidden.
        `inputs_embeds` [T, H] replaces the embedding look-up (vision-language: image features merged in)."""
        if self.has_embed:
            x = inputs_embeds if inputs_embeds is not None else ops.embedding(tokens, self.embed)
            x = self.ps.sp_scatter(x)
        else:
            x = hidden_in
        residual = None
        for layer in self.layers:
            if meta.recompute and torch.is_grad_enabled():
                x, residual = _checkpoint(layer, x, residual, meta)
            else:
                x, residual = layer(x, residual, meta)
        if not self.has_head:
            if getattr(x, "_tp_partial", False):       # a pipeline stage boundary needs the reduced value
                x = self.ps.allreduce_add_rmsnorm(x, residual, self.layers[-1].ln2, self.cfg.rms_eps)[1]
                return x
            return x if residual is None else x + residual
        h, _ = add_rmsnorm_reducing(self.ps, x, residual, self.norm, self.cfg.rms_eps)
        return h

    def global_name(self, name: str) -> str:
        """Parameter name with the model-wide layer index (a pipeline stage numbers its own layers from 0)."""
        lo = self.layer_range[0]
        if lo and name.startswith("layers."):
            _, i, rest = name.split(".", 2)
            return f"layers.{int(i) + lo}.{rest}"
        return name

    def named_parameters_global(self):
        for n, p in self.named_parameters():
            yield self.global_name(n), p

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Full logits (engine sampling / tests). hidden [T,H] → [T,V] fp32 (TP: gathered)."""
        hidden = self.ps.sp_gather(hidden)
        lg = ops.linear_fp32(hidden, self.head_weight())
        return self.ps.tp_all_gather_last(lg)

    def log_probs(self, hidden, targets, temperature: float = 1.0, with_entropy: bool = False):
        """Vocab-parallel log-prob (and entropy) of `targets` from final hidden states."""
        hidden = self.ps.sp_gather(hidden)
        return self.ps.vocab_parallel_logprob(hidden, self.head_weight(), targets, temperature, with_entropy,
                                              self.cfg.vocab_size)


class VirtualStages(nn.Module):
    """The model chunks of one pipeline rank under the interleaved schedule: with `pp` ranks and `vpp` chunks per rank the
    layers are cut into pp · vpp virtual stages and rank r owns stages r, r + pp, r + 2·pp, …  (Megatron's virtual pipeline,
    miles/backends/megatron_utils/model.py:395-411).  Each chunk is a `Qwen3Model` over its layer range: the chunk with layer 0
    embeds, the one with the last layer applies the final norm and owns the head.  Parameter names are global
    (`named_parameters_global`), so checkpoints and weight sync do not see the cut."""

    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype=torch.bfloat16, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg, self.ps, self.dtype = cfg, ps, dtype
        n_virtual = ps.pp_size * ps.vpp_size
        assert cfg.num_layers >= n_virtual, f"{cfg.num_layers} layers cannot fill {n_virtual} virtual stages"
        base, rem = divmod(cfg.num_layers, n_virtual)          # the first `rem` virtual stages take one layer more
        start = [v * base + min(v, rem) for v in range(n_virtual + 1)]
        chunks = []
        for c in range(ps.vpp_size):
            v = c * ps.pp_size + ps.pp_rank
            lo, hi = start[v], start[v + 1]
            chunks.append(Qwen3Model(cfg, ps, dtype=dtype, device=device, seed=seed, layer_range=(lo, hi)))
        self.chunks = nn.ModuleList(chunks)
        self.layer_range = (chunks[0].layer_range[0], chunks[-1].layer_range[1])
        self.has_embed, self.has_head = chunks[0].has_embed, chunks[-1].has_head
        self.num_moe_layers = chunks[0].num_moe_layers

    def forward(self, tokens, meta, hidden_in=None, inputs_embeds=None, chunk: int = 0):
        return self.chunks[chunk](tokens, meta, hidden_in=hidden_in, inputs_embeds=inputs_embeds)

    def global_name(self, name: str) -> str:
        if name.startswith("chunks."):
            _, c, rest = name.split(".", 2)
            return self.chunks[int(c)].global_name(rest)
        return name

    def named_parameters_global(self):
        for n, p in self.named_parameters():
            yield self.global_name(n), p

    def head_weight(self):
        return self.chunks[-1].head_weight()

    def logits(self, hidden):
        return self.chunks[-1].logits(hidden)

    def log_probs(self, hidden, targets, temperature: float = 1.0, with_entropy: bool = False):
        return self.chunks[-1].log_probs(hidden, targets, temperature, with_entropy)


def _checkpoint(layer, x, residual, meta):
    from torch.utils.checkpoint import checkpoint

    if residual is None:
        return checkpoint(lambda a: layer(a, None, meta), x, use_reentrant=False)
    return checkpoint(lambda a, r: layer(a, r, meta), x, residual, use_reentrant=False)


def shard_qkv(full: torch.Tensor, cfg: ModelConfig, rank: int, tp: int) -> torch.Tensor:
    """Slice a [q;k;v]-stacked tensor (dim 0) by heads for one TP rank."""
    if tp == 1:
        return full
    q, k, v = full.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
    return torch.cat([q.chunk(tp, 0)[rank], k.chunk(tp, 0)[rank], v.chunk(tp, 0)[rank]], 0).contiguous()


def unshard_qkv(parts: list[torch.Tensor], cfg: ModelConfig) -> torch.Tensor:
    tp = len(parts)
    qs, ks, vs = [], [], []
    for p in parts:
        q, k, v = p.split([cfg.q_size // tp, cfg.kv_size // tp, cfg.kv_size // tp], dim=0)
        qs.append(q), ks.append(k), vs.append(v)
    return torch.cat(qs + ks + vs, 0)


def build_model(cfg: ModelConfig, ps: ParallelState | None = None, dtype=torch.bfloat16, device="cpu",
                seed: int = 0) -> Qwen3Model:
    ps = ps or ParallelState.single()
    if getattr(cfg, "family", "qwen3") != "qwen3":
        from .families import build_family_model      # latent / sparse / linear attention, shared experts, hyper-connections

        return build_family_model(cfg, ps, dtype=dtype, device=device, seed=seed)
    layer_range = None
    if ps.pp_size > 1 and getattr(ps, "vpp_size", 1) > 1:
        return VirtualStages(cfg, ps, dtype=dtype, device=device, seed=seed)
    if ps.pp_size > 1:
        per = math.ceil(cfg.num_layers / ps.pp_size)
        layer_range = (ps.pp_rank * per, min(cfg.num_layers, (ps.pp_rank + 1) * per))
    return Qwen3Model(cfg, ps, dtype=dtype, device=device, seed=seed, layer_range=layer_range)
