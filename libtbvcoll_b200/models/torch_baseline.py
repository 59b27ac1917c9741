"""The path this library replaces, written with stock PyTorch only: cuBLAS GEMMs
(``torch.matmul``), ``torch.distributed`` (NCCL on GPUs, gloo on CPU) all-reduce after the
row-parallel projections, PyTorch attention over a contiguous KV cache, greedy sampling.
It is (a) the live baseline the benchmarks compare against — the reference's own baseline
is vLLM + NCCL/RCCL (reports/10_tp_custom_allreduce.md:13-16) — and (b) the numerics oracle
for the sm_100a engine on small shapes.  None of this repository's kernels are used here.
Arithmetic follows HF Llama in bf16 op by op.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..ops import reference as ref
from ..ops import rope_cos_sin
from .config import ModelConfig


class TorchLlamaTP:
    def __init__(self, cfg: ModelConfig, rank: int, world: int, weights: Dict[str, torch.Tensor], device, max_batch: int,
                 max_seq_len: int, group=None):
        """``weights``: ``shard_for_rank(..., interleave_gate_up=False)``."""
        self.cfg, self.rank, self.world, self.w, self.device, self.group = cfg, rank, world, weights, torch.device(device), group
        self.nq = cfg.num_heads // world
        self.nkv = cfg.kv_heads_per_rank(world)
        self.D = cfg.head_dim
        self.vpr = cfg.vocab_size // world
        dt = weights["embed"].dtype
        self.k = [torch.zeros(max_batch, max_seq_len, self.nkv, self.D, dtype=dt, device=self.device) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(max_batch, max_seq_len, self.nkv, self.D, dtype=dt, device=self.device) for _ in range(cfg.num_layers)]
        self.cos_sin = rope_cos_sin(self.D, cfg.max_position, cfg.rope_theta, self.device, cfg.rope_scaling)
        self.all_reduces = 0

    def _ar(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            torch.distributed.all_reduce(x, group=self.group)
            self.all_reduces += 1
        return x

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, start: int) -> torch.Tensor:
        """ids, positions: [B, T] (the same T for every row; rows start at cache index ``start``).
        Returns full-vocab logits of the last position [B, V] (fp32)."""
        cfg, w = self.cfg, self.w
        B, T = ids.shape
        local = ids - self.rank * self.vpr
        mine = (local >= 0) & (local < self.vpr)
        h = F.embedding(local.clamp(0, self.vpr - 1), w["embed"]) * mine[..., None].to(w["embed"].dtype)
        h = self._ar(h)
        pos_flat = positions.reshape(-1)
        scale = 1.0 / math.sqrt(self.D)
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            x = ref.rmsnorm(h, w[p + "input_norm"], cfg.rms_eps)
            qkv = F.linear(x, w[p + "qkv.weight"], w.get(p + "qkv.bias")).view(B * T, self.nq + 2 * self.nkv, self.D)
            qk = ref.rope(qkv[:, : self.nq + self.nkv], pos_flat, self.cos_sin)
            q = qk[:, : self.nq].view(B, T, self.nq, self.D)
            self.k[l][:B, start:start + T] = qk[:, self.nq:].view(B, T, self.nkv, self.D)
            self.v[l][:B, start:start + T] = qkv[:, self.nq + self.nkv:].view(B, T, self.nkv, self.D)
            kk = self.k[l][:B, : start + T].transpose(1, 2)
            vv = self.v[l][:B, : start + T].transpose(1, 2)
            g = self.nq // self.nkv
            if g > 1:
                kk, vv = kk.repeat_interleave(g, 1), vv.repeat_interleave(g, 1)
            mask = None
            if T > 1:
                qi = torch.arange(T, device=ids.device)[:, None] + start
                mask = torch.arange(start + T, device=ids.device)[None, :] <= qi
            a = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask, scale=scale)
            a = a.transpose(1, 2).reshape(B, T, self.nq * self.D)
            h = h + self._ar(F.linear(a, w[p + "o.weight"]))
            x = ref.rmsnorm(h, w[p + "post_norm"], cfg.rms_eps)
            gu = F.linear(x, w[p + "gate_up.weight"])
            h = h + self._ar(F.linear(ref.silu_mul(gu), w[p + "down.weight"]))
        x = ref.rmsnorm(h[:, -1], w["norm"], cfg.rms_eps)
        logits = F.linear(x, w["lm_head"])
        if self.world > 1:
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            torch.distributed.all_gather(parts, logits, group=self.group)
            logits = torch.cat(parts, -1)
        return logits.float()

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int) -> List[List[int]]:
        """Greedy; all prompts must have the same length (the benchmark's shape)."""
        B, L = len(prompts), len(prompts[0])
        assert all(len(p) == L for p in prompts)
        ids = torch.tensor(prompts, dtype=torch.int64, device=self.device)
        pos = torch.arange(L, device=self.device, dtype=torch.int32)[None].expand(B, L)
        _, tok = ref.argmax_first(self.forward(ids, pos, 0))
        outs = [[int(t)] for t in tok]
        for s in range(max_new_tokens - 1):
            p = torch.full((B, 1), L + s, dtype=torch.int32, device=self.device)
            _, tok = ref.argmax_first(self.forward(tok.view(B, 1), p, L + s))
            for b in range(B):
                outs[b].append(int(tok[b]))
        return outs


class GraphedTorchDecoder:
    """One decode step of ``TorchLlamaTP`` captured in a CUDA graph (what vLLM does for its
    NCCL + cuBLAS path), so the baseline is not penalised by Python/launch overhead."""

    def __init__(self, model: TorchLlamaTP, batch: int, start: int):
        self.m, self.B = model, batch
        dev = model.device
        self.ids = torch.zeros(batch, 1, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(batch, 1, dtype=torch.int32, device=dev)
        self.out = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.start = start
        self.graph: Optional[torch.cuda.CUDAGraph] = None

    def _step(self):
        # a fixed cache window keeps shapes static under capture: attend over [0, start] with
        # the new token written at index `start` (the timing shape of a step at that context)
        logits = self.m.forward(self.ids, self.pos, self.start)
        self.out.copy_(logits.argmax(-1))

    @torch.no_grad()
    def capture(self):
        s = torch.cuda.Stream(device=self.m.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._step()
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self._step()
        torch.cuda.current_stream().wait_stream(s)
        self.graph = g

    def replay(self):
        self.graph.replay()
