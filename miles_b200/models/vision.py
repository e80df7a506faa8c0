"""Vision tower and multimodal merge for vision-language policies (the Qwen-VL layout).

An image (or video frame group) arrives as a sequence of flattened patches [N, C·p·p] with its grid (t, h, w).  The tower
is a ViT over those patches: linear patch embedding, pre-norm blocks of bidirectional attention restricted to one image
(`cu_seqlens` over images, the same varlen attention kernel as the language model with `causal=False`) with a
two-dimensional rotary embedding (half of every head rotates by the patch row, half by its column), SwiGLU MLPs, and a
patch merger that concatenates `merge × merge` neighbouring patches and projects them to the language model's width.
`merge_multimodal` puts the merged features at the positions of the image placeholder token, after which the language
model runs on `inputs_embeds` as usual.

Reference behaviour: the vision/audio towers of miles_plugins/models/qwen3_vl (layer specs) and the "multimodal merge" of
miles/backends/megatron_utils/data.py (get_batch); here they are plain modules on this package's ops, so the tower
trains with the policy (its parameters join the same optimizer) or stays frozen (`requires_grad_(False)`).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops


@dataclass(frozen=True)
class VisionConfig:
    patch_size: int = 14
    in_channels: int = 3
    temporal_patch: int = 1
    hidden_size: int = 256
    num_heads: int = 4
    num_layers: int = 2
    ffn_hidden_size: int = 512
    spatial_merge: int = 2
    out_hidden_size: int = 256          # the language model's hidden size
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    init_std: float = 0.02

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch * self.patch_size * self.patch_size

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def patch_positions(grid_thw: torch.Tensor, merge: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Row / column index of every patch and the image boundaries, for patches ordered so that each `merge × merge` window
    is contiguous (the order image processors emit, which lets the merger be a reshape).  grid_thw: int [n_images, 3]."""
    rows, cols, cu = [], [], [0]
    for t, h, w in grid_thw.tolist():
        assert h % merge == 0 and w % merge == 0, "grid must be a multiple of the spatial merge size"
        r = torch.arange(h).view(h // merge, merge, 1, 1).expand(h // merge, merge, w // merge, merge)
        c = torch.arange(w).view(1, 1, w // merge, merge).expand(h // merge, merge, w // merge, merge)
        # (h/m, m, w/m, m) → (h/m, w/m, m, m): windows contiguous
        r = r.permute(0, 2, 1, 3).reshape(-1)
        c = c.permute(0, 2, 1, 3).reshape(-1)
        for _ in range(t):
            rows.append(r)
            cols.append(c)
            cu.append(cu[-1] + h * w)
    return torch.cat(rows).to(torch.int32), torch.cat(cols).to(torch.int32), torch.tensor(cu, dtype=torch.int32)


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device, gen: torch.Generator):
        super().__init__()
        H, F = cfg.hidden_size, cfg.ffn_hidden_size

        def w(*shape):
            return nn.Parameter((cfg.init_std * torch.randn(*shape, generator=gen)).to(dtype=dtype, device=device))

        self.cfg = cfg
        self.ln1 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.wqkv = w(3 * H, H)
        self.wo = w(H, H)
        self.ln2 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.w13 = w(2 * F, H)
        self.w2 = w(H, F)

    def forward(self, x, rows, cols, cu, max_len):
        cfg = self.cfg
        N, nh, d = x.shape[0], cfg.num_heads, cfg.head_dim
        h = ops.rmsnorm(x, self.ln1, cfg.rms_eps)
        q, k, v = ops.linear(h, self.wqkv).view(N, 3, nh, d).unbind(1)
        # 2-D rotary: the first half of each head follows the patch row, the second half its column
        half = d // 2
        q = torch.cat([ops.rope(q[..., :half].contiguous(), rows, cfg.rope_theta),
                       ops.rope(q[..., half:].contiguous(), cols, cfg.rope_theta)], dim=-1)
        k = torch.cat([ops.rope(k[..., :half].contiguous(), rows, cfg.rope_theta),
                       ops.rope(k[..., half:].contiguous(), cols, cfg.rope_theta)], dim=-1)
        o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu, max_len, causal=False)
        x = x + ops.linear(o.reshape(N, nh * d), self.wo)
        h = ops.rmsnorm(x, self.ln2, cfg.rms_eps)
        return x + ops.linear(ops.swiglu(ops.linear(h, self.w13)), self.w2)


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=torch.bfloat16, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator().manual_seed(seed + 7919)
        H, m2 = cfg.hidden_size, cfg.spatial_merge ** 2

        def w(*shape):
            return nn.Parameter((cfg.init_std * torch.randn(*shape, generator=gen)).to(dtype=dtype, device=device))

        self.patch_embed = w(H, cfg.patch_dim)
        self.blocks = nn.ModuleList([VisionBlock(cfg, dtype, device, gen) for _ in range(cfg.num_layers)])
        self.merger_norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.merger_fc1 = w(m2 * H, m2 * H)
        self.merger_fc2 = w(cfg.out_hidden_size, m2 * H)

    def forward(self, patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """patches [N, C·tp·p·p] (windows of `merge × merge` contiguous), grid_thw int [n_images, 3] →
        features [N / merge², out_hidden_size], one row per image placeholder token."""
        cfg = self.cfg
        rows, cols, cu = patch_positions(grid_thw.cpu(), cfg.spatial_merge)
        assert patches.shape[0] == int(cu[-1]), f"{patches.shape[0]} patches for grids that hold {int(cu[-1])}"
        dev = patches.device
        rows, cols, cu = rows.to(dev), cols.to(dev), cu.to(dev)
        max_len = int((cu[1:] - cu[:-1]).max())
        x = ops.linear(patches.to(self.patch_embed.dtype), self.patch_embed)
        for blk in self.blocks:
            x = blk(x, rows, cols, cu, max_len)
        x = ops.rmsnorm(x, self.merger_norm, cfg.rms_eps)
        x = x.view(-1, cfg.spatial_merge ** 2 * cfg.hidden_size)
        return ops.linear(torch.nn.functional.gelu(ops.linear(x, self.merger_fc1)), self.merger_fc2)


def merge_multimodal(embeds: torch.Tensor, tokens: torch.Tensor, image_token_id: int, feats: torch.Tensor) -> torch.Tensor:
    """Rows of `embeds` [T, H] whose token is the image placeholder are replaced, in order, by `feats` [n, H]
    (differentiable in both)."""
    mask = tokens.long() == image_token_id
    n = int(mask.sum())
    assert n == feats.shape[0], f"{n} image placeholder tokens for {feats.shape[0]} vision features"
    idx = mask.nonzero().flatten()
    return embeds.index_copy(0, idx, feats.to(embeds.dtype))


class VisionLanguageModel(nn.Module):
    """A language model of this package with a vision tower in front: `forward` takes the packed token stream plus the
    patches of all its images and returns what the language model returns."""

    def __init__(self, lm, tower: VisionTower, image_token_id: int):
        super().__init__()
        assert tower.cfg.out_hidden_size == lm.cfg.hidden_size
        self.lm, self.tower, self.image_token_id = lm, tower, int(image_token_id)
        self.cfg = lm.cfg

    def forward(self, tokens, meta, patches: torch.Tensor | None = None, grid_thw: torch.Tensor | None = None):
        if patches is None or patches.numel() == 0:
            return self.lm(tokens, meta)
        embeds = ops.embedding(tokens, self.lm.embed)
        embeds = merge_multimodal(embeds, tokens, self.image_token_id, self.tower(patches, grid_thw))
        return self.lm(tokens, meta, inputs_embeds=embeds)

    def logits(self, hidden):
        return self.lm.logits(hidden)

    def log_probs(self, hidden, targets, temperature: float = 1.0, with_entropy: bool = False):
        return self.lm.log_probs(hidden, targets, temperature, with_entropy)
