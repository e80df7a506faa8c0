"""Model architecture descriptions.

One dataclass covers the Qwen2/Qwen3 dense family and the Qwen3-MoE family (softmax top-k router,
per-expert SwiGLU FFN).  Presets mirror the shape flags the reference passes to Megatron
(scripts/models/qwen3-4B.py, qwen3-32B.py, qwen3-30B-A3B.py:9-45) and the HF `config.json` keys.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, replace


@dataclass(frozen=True)
class ModelConfig:
    name: str = "tiny"
    vocab_size: int = 2048
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    ffn_hidden_size: int = 688
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    qkv_bias: bool = False
    tie_embeddings: bool = False
    # MoE (num_experts == 0 → dense)
    num_experts: int = 0
    moe_topk: int = 0
    moe_ffn_hidden_size: int = 0
    moe_norm_topk_prob: bool = True
    first_k_dense: int = 0
    max_position: int = 40960
    init_std: float = 0.02

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    def layer_is_moe(self, layer: int) -> bool:
        return self.is_moe and layer >= self.first_k_dense

    def num_params(self, active_only: bool = False) -> int:
        h = self.hidden_size
        attn = h * self.qkv_size + self.q_size * h + (2 * self.head_dim if self.qk_norm else 0)
        if self.qkv_bias:
            attn += self.qkv_size
        total = 0
        for l in range(self.num_layers):
            total += attn + 2 * h
            if self.layer_is_moe(l):
                e = self.moe_topk if active_only else self.num_experts
                total += e * 3 * h * self.moe_ffn_hidden_size + h * self.num_experts
            else:
                total += 3 * h * self.ffn_hidden_size
        total += h + self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return total

    def flops_per_token(self, seq_len: int, backward: bool = True) -> float:
        """Matmul FLOPs per token (2·active params, causal attention 2·2·s/2·q_size), ×3 with backward."""
        dense = 2.0 * (self.num_params(active_only=True) - self.vocab_size * self.hidden_size * (0 if self.tie_embeddings else 1))
        attn = self.num_layers * 2.0 * 2.0 * (seq_len / 2.0) * self.q_size
        f = dense + attn
        return f * (3.0 if backward else 1.0)

    def to_hf_config(self) -> dict:
        d = {
            "architectures": ["Qwen3MoeForCausalLM" if self.is_moe else "Qwen3ForCausalLM"],
            "model_type": "qwen3_moe" if self.is_moe else "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.ffn_hidden_size,
            "rms_norm_eps": self.rms_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_embeddings,
            "attention_bias": self.qkv_bias,
            "max_position_embeddings": self.max_position,
            "torch_dtype": "bfloat16",
        }
        if self.is_moe:
            d.update(
                num_experts=self.num_experts,
                num_experts_per_tok=self.moe_topk,
                moe_intermediate_size=self.moe_ffn_hidden_size,
                norm_topk_prob=self.moe_norm_topk_prob,
                mlp_only_layers=list(range(self.first_k_dense)),
                decoder_sparse_step=1,
            )
        return d

    @staticmethod
    def from_hf_config(cfg: dict | str) -> "ModelConfig":
        if isinstance(cfg, str):
            path = os.path.join(cfg, "config.json") if os.path.isdir(cfg) else cfg
            with open(path) as f:
                cfg = json.load(f)
        mt = cfg.get("model_type", "qwen3")
        heads = cfg["num_attention_heads"]
        head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads
        moe = "moe" in mt
        return ModelConfig(
            name=cfg.get("_name_or_path", mt) or mt,
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            num_layers=cfg["num_hidden_layers"],
            num_heads=heads,
            num_kv_heads=cfg.get("num_key_value_heads", heads),
            head_dim=head_dim,
            ffn_hidden_size=cfg.get("intermediate_size", 0),
            rms_eps=cfg.get("rms_norm_eps", 1e-6),
            rope_theta=cfg.get("rope_theta", 1e6),
            qk_norm=mt.startswith("qwen3"),
            qkv_bias=cfg.get("attention_bias", mt == "qwen2"),
            tie_embeddings=cfg.get("tie_word_embeddings", False),
            num_experts=cfg.get("num_experts", 0) if moe else 0,
            moe_topk=cfg.get("num_experts_per_tok", 0) if moe else 0,
            moe_ffn_hidden_size=cfg.get("moe_intermediate_size", 0) if moe else 0,
            moe_norm_topk_prob=cfg.get("norm_topk_prob", True),
            first_k_dense=len(cfg.get("mlp_only_layers", []) or []),
            max_position=cfg.get("max_position_embeddings", 40960),
        )

    def save(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump(self.to_hf_config(), f, indent=2)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)

    def asdict(self) -> dict:
        return asdict(self)


PRESETS: dict[str, ModelConfig] = {
    # CPU plumbing model of the tiny GRPO run
    "tiny": ModelConfig(),
    "tiny-moe": ModelConfig(name="tiny-moe", num_experts=8, moe_topk=2, moe_ffn_hidden_size=128),
    "qwen3-0.6B": ModelConfig(
        name="qwen3-0.6B", vocab_size=151936, hidden_size=1024, num_layers=28, num_heads=16,
        num_kv_heads=8, head_dim=128, ffn_hidden_size=3072, tie_embeddings=True),
    "qwen3-4B": ModelConfig(
        name="qwen3-4B", vocab_size=151936, hidden_size=2560, num_layers=36, num_heads=32,
        num_kv_heads=8, head_dim=128, ffn_hidden_size=9728),
    "qwen3-8B": ModelConfig(
        name="qwen3-8B", vocab_size=151936, hidden_size=4096, num_layers=36, num_heads=32,
        num_kv_heads=8, head_dim=128, ffn_hidden_size=12288),
    "qwen3-32B": ModelConfig(
        name="qwen3-32B", vocab_size=151936, hidden_size=5120, num_layers=64, num_heads=64,
        num_kv_heads=8, head_dim=128, ffn_hidden_size=25600),
    "qwen3-30B-A3B": ModelConfig(
        name="qwen3-30B-A3B", vocab_size=151936, hidden_size=2048, num_layers=48, num_heads=32,
        num_kv_heads=4, head_dim=128, ffn_hidden_size=6144, num_experts=128, moe_topk=8,
        moe_ffn_hidden_size=768),
    "qwen3-235B-A22B": ModelConfig(
        name="qwen3-235B-A22B", vocab_size=151936, hidden_size=4096, num_layers=94, num_heads=64,
        num_kv_heads=4, head_dim=128, ffn_hidden_size=12288, num_experts=128, moe_topk=8,
        moe_ffn_hidden_size=1536),
    "qwen2.5-0.5B": ModelConfig(
        name="qwen2.5-0.5B", vocab_size=151936, hidden_size=896, num_layers=24, num_heads=14,
        num_kv_heads=2, head_dim=64, ffn_hidden_size=4864, qk_norm=False, qkv_bias=True,
        tie_embeddings=True),
}


def get_config(name_or_path: str) -> ModelConfig:
    if name_or_path not in PRESETS and not os.path.exists(name_or_path):
        from . import families  # noqa: F401  (registers the presets of the other model families)
    if name_or_path in PRESETS:
        return PRESETS[name_or_path]
    if os.path.exists(name_or_path):
        return ModelConfig.from_hf_config(name_or_path)
    raise KeyError(f"unknown model '{name_or_path}'; presets: {sorted(PRESETS)}")
