"""Weights in the HF safetensors layout, sharded for tensor parallelism.

The reference's engine did "TP-sharded weight loading" from an HF model directory
(reports/11_custom_engine.md:12; models are mounted read-only, step3b/node_launch.sh:31).
Here: a reader for ``*.safetensors`` (+ ``model.safetensors.index.json``) that slices each
tensor for one rank, and a seeded random initialiser that yields tensors under the SAME HF
names and shapes, so benchmarks and tests go through the same sharding code as a real
checkpoint.  Sharding: q/k/v/gate/up by output rows (column-parallel), o_proj/down_proj by
input columns (row-parallel), embed_tokens/lm_head by vocabulary rows.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Callable, Dict, Iterable, Optional

import torch

from ..models.config import ModelConfig


def hf_tensor_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    h, d = cfg.hidden_size, cfg.head_dim
    shapes = {"model.embed_tokens.weight": (cfg.vocab_size, h), "model.norm.weight": (h,)}
    if not cfg.tie_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, h)
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes[p + "self_attn.q_proj.weight"] = (cfg.num_heads * d, h)
        shapes[p + "self_attn.k_proj.weight"] = (cfg.num_kv_heads * d, h)
        shapes[p + "self_attn.v_proj.weight"] = (cfg.num_kv_heads * d, h)
        shapes[p + "self_attn.o_proj.weight"] = (h, cfg.num_heads * d)
        if cfg.qkv_bias:
            shapes[p + "self_attn.q_proj.bias"] = (cfg.num_heads * d,)
            shapes[p + "self_attn.k_proj.bias"] = (cfg.num_kv_heads * d,)
            shapes[p + "self_attn.v_proj.bias"] = (cfg.num_kv_heads * d,)
        shapes[p + "mlp.gate_proj.weight"] = (cfg.intermediate_size, h)
        shapes[p + "mlp.up_proj.weight"] = (cfg.intermediate_size, h)
        shapes[p + "mlp.down_proj.weight"] = (h, cfg.intermediate_size)
    return shapes


class RandomSource:
    """Seeded random weights under HF names.  A tensor's values depend only on (seed, name),
    never on the TP degree, so every rank slices the same virtual checkpoint."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.seed, self.device, self.dtype = cfg, seed, torch.device(device), dtype
        self.shapes = hf_tensor_shapes(cfg)

    def names(self) -> Iterable[str]:
        return self.shapes.keys()

    def get(self, name: str) -> torch.Tensor:
        shape = self.shapes[name]
        g = torch.Generator(device=self.device).manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
        if name.endswith("layernorm.weight") or name.endswith("norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=self.device, dtype=torch.float32)
        elif name.endswith(".bias"):
            t = 0.1 * torch.randn(shape, generator=g, device=self.device, dtype=torch.float32)
        else:
            t = 0.02 * torch.randn(shape, generator=g, device=self.device, dtype=torch.float32)
        return t.to(self.dtype)


class SafetensorsSource:
    """An HF checkpoint directory (single file or sharded with an index)."""

    def __init__(self, path: str, device="cpu", dtype=torch.bfloat16):
        from safetensors import safe_open
        self.device, self.dtype = device, dtype
        self._open = safe_open
        idx = os.path.join(path, "model.safetensors.index.json")
        self.where: Dict[str, str] = {}
        if os.path.exists(idx):
            with open(idx) as f:
                for k, v in json.load(f)["weight_map"].items():
                    self.where[k] = os.path.join(path, v)
        else:
            files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
            if not files:
                raise FileNotFoundError(f"no .safetensors under {path}")
            for fn in files:
                with safe_open(os.path.join(path, fn), framework="pt") as f:
                    for k in f.keys():
                        self.where[k] = os.path.join(path, fn)

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def get(self, name: str) -> torch.Tensor:
        with self._open(self.where[name], framework="pt", device="cpu") as f:
            return f.get_tensor(name).to(self.dtype).to(self.device)

    def get_rows(self, name: str, r0: int, r1: int) -> torch.Tensor:
        """Rows [r0, r1) without reading the rest of the tensor."""
        with self._open(self.where[name], framework="pt", device="cpu") as f:
            return f.get_slice(name)[r0:r1].to(self.dtype).to(self.device)


def save_hf_checkpoint(source, path: str, max_shard_bytes: int = 1 << 30) -> None:
    """Write every tensor of ``source`` as an HF-style sharded safetensors checkpoint."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for n in source.names():
        t = source.get(n).cpu().contiguous()
        if cur and cur_bytes + t.numel() * t.element_size() > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[n] = t
        cur_bytes += t.numel() * t.element_size()
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn))
        for n in sh:
            weight_map[n] = fn
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)


def _rows(source, name: str, r0: int, r1: int) -> torch.Tensor:
    if hasattr(source, "get_rows"):
        return source.get_rows(name, r0, r1)
    return source.get(name)[r0:r1]


def shard_for_rank(cfg: ModelConfig, source, rank: int, tp: int, device, interleave_gate_up: bool = True) -> Dict[str, torch.Tensor]:
    """Per-rank tensors, fused the way the kernels consume them:
    ``layers.{l}.qkv.weight`` [(nq+2nkv)*D / tp', hidden], ``layers.{l}.qkv.bias``,
    ``layers.{l}.o.weight`` [hidden, nq*D/tp], ``layers.{l}.gate_up.weight`` [2*I/tp, hidden]
    (rows interleaved gate_i, up_i when ``interleave_gate_up``; otherwise [gate | up]),
    ``layers.{l}.down.weight`` [hidden, I/tp], the two norm weights per layer, ``embed``
    [V/tp, hidden], ``lm_head`` [V/tp, hidden], ``norm``."""
    cfg.check_tp(tp)
    d = cfg.head_dim
    nq = cfg.num_heads // tp
    nkv = cfg.kv_heads_per_rank(tp)
    # kv heads are split while there are at least `tp` of them, replicated beyond that
    kv0 = rank * nkv if cfg.num_kv_heads >= tp else rank // (tp // cfg.num_kv_heads)
    ipr = cfg.intermediate_size // tp
    vpr = cfg.vocab_size // tp
    out: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)

    def put(k, t):
        out[k] = t.to(dev).contiguous()

    put("embed", _rows(source, "model.embed_tokens.weight", rank * vpr, (rank + 1) * vpr))
    head = "model.embed_tokens.weight" if cfg.tie_embeddings else "lm_head.weight"
    put("lm_head", _rows(source, head, rank * vpr, (rank + 1) * vpr))
    put("norm", source.get("model.norm.weight"))
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        q = _rows(source, p + "self_attn.q_proj.weight", rank * nq * d, (rank + 1) * nq * d)
        k = _rows(source, p + "self_attn.k_proj.weight", kv0 * d, (kv0 + nkv) * d)
        v = _rows(source, p + "self_attn.v_proj.weight", kv0 * d, (kv0 + nkv) * d)
        put(f"layers.{l}.qkv.weight", torch.cat((q, k, v), 0))
        if cfg.qkv_bias:
            qb = _rows(source, p + "self_attn.q_proj.bias", rank * nq * d, (rank + 1) * nq * d)
            kb = _rows(source, p + "self_attn.k_proj.bias", kv0 * d, (kv0 + nkv) * d)
            vb = _rows(source, p + "self_attn.v_proj.bias", kv0 * d, (kv0 + nkv) * d)
            put(f"layers.{l}.qkv.bias", torch.cat((qb, kb, vb), 0))
        put(f"layers.{l}.o.weight", source.get(p + "self_attn.o_proj.weight")[:, rank * nq * d:(rank + 1) * nq * d])
        g = _rows(source, p + "mlp.gate_proj.weight", rank * ipr, (rank + 1) * ipr)
        u = _rows(source, p + "mlp.up_proj.weight", rank * ipr, (rank + 1) * ipr)
        if interleave_gate_up:
            put(f"layers.{l}.gate_up.weight", torch.stack((g, u), 1).reshape(2 * ipr, cfg.hidden_size))
        else:
            put(f"layers.{l}.gate_up.weight", torch.cat((g, u), 0))
        put(f"layers.{l}.down.weight", source.get(p + "mlp.down_proj.weight")[:, rank * ipr:(rank + 1) * ipr])
        put(f"layers.{l}.input_norm", source.get(p + "input_layernorm.weight"))
        put(f"layers.{l}.post_norm", source.get(p + "post_attention_layernorm.weight"))
    return out
