"""Audio tower: log-mel frames of variable-length clips → one feature row per audio placeholder token of the language model.

The multimodal families of the reference carry audio next to vision (tower modules inside their Megatron layer specs,
miles_plugins/models/*: "vision/audio towers").  The shape here is the usual speech encoder: two 1-D convolutions over
time (kernel 3; the second with stride 2) with GELU, sinusoidal positions, bidirectional transformer blocks whose attention
stays inside each clip (packed variable-length attention, the same kernel as the vision tower), a final norm, and a
projector that pools `pool` neighbouring frames into one row of the language model's width.  Clips are packed along time:
`features` [Σ frames, n_mels] with `clip_frames` [n_clips]; a clip of f frames yields ⌈⌈f / 2⌉ / pool⌉ rows.
`AudioLanguageModel` merges those rows into the token stream at the audio placeholder id, like the vision wrapper does for
image tokens (`models/vision.py`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .vision import merge_multimodal


@dataclass
class AudioConfig:
    n_mels: int = 80
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    ffn_hidden_size: int = 512
    pool: int = 2                      # frames (after the stride-2 convolution) pooled into one output row
    out_hidden_size: int = 256
    rms_eps: float = 1e-6
    init_std: float = 0.02
    max_positions: int = 3000

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def output_rows(clip_frames: torch.Tensor, pool: int) -> torch.Tensor:
    """Rows the tower emits per clip: stride-2 convolution, then pooling (both round up)."""
    half = (clip_frames + 1) // 2
    return (half + pool - 1) // pool


def _sinusoids(n: int, dim: int, device) -> torch.Tensor:
    inv = torch.exp(-math.log(10000.0) * torch.arange(dim // 2, device=device, dtype=torch.float32) / max(dim // 2 - 1, 1))
    t = torch.arange(n, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=-1)


class AudioBlock(nn.Module):
    def __init__(self, cfg: AudioConfig, dtype, device, gen: torch.Generator):
        super().__init__()
        H, Fh = cfg.hidden_size, cfg.ffn_hidden_size

        def w(*shape):
            return nn.Parameter((cfg.init_std * torch.randn(*shape, generator=gen)).to(dtype=dtype, device=device))

        self.cfg = cfg
        self.ln1 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.wqkv, self.wo = w(3 * H, H), w(H, H)
        self.ln2 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.w1, self.w2 = w(Fh, H), w(H, Fh)

    def forward(self, x, cu, max_len):
        cfg = self.cfg
        N, nh, d = x.shape[0], cfg.num_heads, cfg.head_dim
        q, k, v = ops.linear(ops.rmsnorm(x, self.ln1, cfg.rms_eps), self.wqkv).view(N, 3, nh, d).unbind(1)
        o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu, max_len, causal=False)
        x = x + ops.linear(o.reshape(N, nh * d), self.wo)
        return x + ops.linear(F.gelu(ops.linear(ops.rmsnorm(x, self.ln2, cfg.rms_eps), self.w1)), self.w2)


class AudioTower(nn.Module):
    def __init__(self, cfg: AudioConfig, dtype=torch.bfloat16, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator().manual_seed(seed + 104729)
        H = cfg.hidden_size

        def w(*shape):
            return nn.Parameter((cfg.init_std * torch.randn(*shape, generator=gen)).to(dtype=dtype, device=device))

        self.conv1_w, self.conv1_b = w(H, cfg.n_mels, 3), nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.conv2_w, self.conv2_b = w(H, H, 3), nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([AudioBlock(cfg, dtype, device, gen) for _ in range(cfg.num_layers)])
        self.norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.proj1, self.proj2 = w(cfg.pool * H, cfg.pool * H), w(cfg.out_hidden_size, cfg.pool * H)

    def forward(self, features: torch.Tensor, clip_frames: torch.Tensor) -> torch.Tensor:
        """features [Σ frames, n_mels], clip_frames int [n_clips] → [Σ output_rows, out_hidden_size]."""
        cfg = self.cfg
        frames = [int(f) for f in clip_frames.tolist()]
        assert features.shape[0] == sum(frames), f"{features.shape[0]} frames for clips that hold {sum(frames)}"
        dtype, dev = self.conv1_w.dtype, features.device
        pieces, lens, at = [], [], 0
        for f in frames:                                   # the convolutions see one clip at a time: no leakage across clips
            x = features[at:at + f].to(dtype).t()[None]                                        # [1, n_mels, f]
            x = F.gelu(F.conv1d(x, self.conv1_w, self.conv1_b, padding=1))
            x = F.gelu(F.conv1d(x, self.conv2_w, self.conv2_b, stride=2, padding=1))[0].t()    # [⌈f/2⌉, H]
            x = x + _sinusoids(x.shape[0], cfg.hidden_size, dev).to(dtype)
            pieces.append(x)
            lens.append(x.shape[0])
            at += f
        x = torch.cat(pieces) if pieces else features.new_zeros(0, cfg.hidden_size, dtype=dtype)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()) if lens else [0], dtype=torch.int32, device=dev)
        max_len = max(lens, default=0)
        for blk in self.blocks:
            x = blk(x, cu, max_len)
        x = ops.rmsnorm(x, self.norm, cfg.rms_eps)
        out, at = [], 0
        for n in lens:                                     # pool neighbouring frames of one clip (zero-padded to a multiple)
            c = x[at:at + n]
            pad = (-n) % cfg.pool
            if pad:
                c = torch.cat([c, c.new_zeros(pad, cfg.hidden_size)])
            out.append(c.view(-1, cfg.pool * cfg.hidden_size))
            at += n
        y = torch.cat(out) if out else x.new_zeros(0, cfg.pool * cfg.hidden_size)
        return ops.linear(F.gelu(ops.linear(y, self.proj1)), self.proj2)


class AudioLanguageModel(nn.Module):
    """A language model of this package with an audio tower in front: `forward` takes the packed token stream plus the
    log-mel frames of all its clips and returns what the language model returns."""

    def __init__(self, lm, tower: AudioTower, audio_token_id: int):
        super().__init__()
        assert tower.cfg.out_hidden_size == lm.cfg.hidden_size
        self.lm, self.tower, self.audio_token_id = lm, tower, int(audio_token_id)
        self.cfg = lm.cfg

    def forward(self, tokens, meta, audio_features: torch.Tensor | None = None, clip_frames: torch.Tensor | None = None):
        if audio_features is None or audio_features.numel() == 0:
            return self.lm(tokens, meta)
        embeds = ops.embedding(tokens, self.lm.embed)
        embeds = merge_multimodal(embeds, tokens, self.audio_token_id, self.tower(audio_features, clip_frames))
        return self.lm(tokens, meta, inputs_embeds=embeds)

    def logits(self, hidden):
        return self.lm.logits(hidden)

    def log_probs(self, hidden, targets, temperature: float = 1.0, with_entropy: bool = False):
        return self.lm.log_probs(hidden, targets, temperature, with_entropy)
