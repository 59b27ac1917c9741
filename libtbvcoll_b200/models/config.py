"""Model shapes.  The reference serves Qwen2.5-7B-Instruct through vLLM
(step3b/run_vllm_tp.sh:9-10); the benchmark configurations of this repository are
Llama-3-8B- and Llama-3-70B-shaped.  All are the same decoder family (RMSNorm, RoPE,
GQA, SiLU-gated MLP); Qwen2 adds a bias on the q/k/v projections."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class ModelConfig:
    name: str = "llama3-8b"
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    vocab_size: int = 128256
    rope_theta: float = 5e5
    rms_eps: float = 1e-5
    max_position: int = 8192
    qkv_bias: bool = False
    tie_embeddings: bool = False
    rope_scaling: Optional[dict] = field(default=None)

    def check_tp(self, tp: int) -> None:
        if self.num_heads % tp or self.intermediate_size % tp or self.vocab_size % tp:
            raise ValueError(f"{self.name}: heads/intermediate/vocab not divisible by tp={tp}")
        if self.num_kv_heads % tp and tp % self.num_kv_heads:
            raise ValueError(f"{self.name}: kv heads {self.num_kv_heads} incompatible with tp={tp}")
        if self.head_dim != 128:
            raise ValueError("the attention kernels are written for head_dim 128")

    def kv_heads_per_rank(self, tp: int) -> int:
        return max(1, self.num_kv_heads // tp)  # replicated when tp > kv heads

    def param_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        qkv = h * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        per_layer = qkv + self.num_heads * self.head_dim * h + 3 * h * i + 2 * h
        return self.num_layers * per_layer + v * h * (1 if self.tie_embeddings else 2) + h


PRESETS = {
    "llama3-8b": ModelConfig(),
    "llama3-70b": ModelConfig(name="llama3-70b", hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8,
                              intermediate_size=28672),
    "qwen2.5-7b": ModelConfig(name="qwen2.5-7b", hidden_size=3584, num_layers=28, num_heads=28, num_kv_heads=4,
                              intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_eps=1e-6, max_position=32768,
                              qkv_bias=True),
    # small shapes for tests: every dimension still meets the kernels' divisibility rules
    "tiny": ModelConfig(name="tiny", hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, intermediate_size=1024,
                        vocab_size=2048, max_position=512),
    "tiny-bias": ModelConfig(name="tiny-bias", hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=4, intermediate_size=1024,
                             vocab_size=2048, max_position=512, qkv_bias=True, rope_theta=1e4),
}


def get_config(name: str) -> ModelConfig:
    import copy
    return copy.deepcopy(PRESETS[name])


def from_hf_config(path: str) -> ModelConfig:
    """Read an HF ``config.json`` (Llama / Qwen2 families)."""
    with open(path) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    return ModelConfig(
        name=c.get("_name_or_path", c.get("model_type", "hf")),
        hidden_size=c["hidden_size"], num_layers=c["num_hidden_layers"], num_heads=heads,
        num_kv_heads=c.get("num_key_value_heads", heads), head_dim=c.get("head_dim", c["hidden_size"] // heads),
        intermediate_size=c["intermediate_size"], vocab_size=c["vocab_size"], rope_theta=c.get("rope_theta", 1e4),
        rms_eps=c.get("rms_norm_eps", 1e-5), max_position=c.get("max_position_embeddings", 8192),
        qkv_bias=c.get("attention_bias", c.get("model_type") == "qwen2"), tie_embeddings=c.get("tie_word_embeddings", False),
        rope_scaling=c.get("rope_scaling"))
