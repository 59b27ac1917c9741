"""Llama-family decoder (Llama-3 8B/70B shapes, Qwen2 with qkv bias) for one tensor-parallel
rank, built only from the hand-written sm_100a operators and the tbvcoll collectives.

This is the model layer the reference documents but does not ship ("TP=1/2 decode engine:
weight TP sharding, RoPE, GQA, KV cache, greedy", reports/11_custom_engine.md:10-20), with
the weight fusions it names (q/k/v -> qkv, gate/up -> gate_up, :38).  Per layer:

    qkv GEMM (RoPE + KV-cache write in its epilogue) -> paged attention -> o_proj GEMM (partial sums)
    -> all-reduce + residual + RMSNorm (ONE kernel)  -> gate_up GEMM with SiLU-mul epilogue
    -> down_proj GEMM (partial sums) -> all-reduce + residual + next RMSNorm (ONE kernel)

i.e. 7 launches per layer with TP > 1 (5 GEMM / attention kernels and the two fused collectives the
reference's hook intercepts as plain all-reduces, 2 per layer; step3b/vllm_tp_bench.py:87-124), chained by
programmatic dependent launch so that each GEMM streams its weights while the collective before it runs.
``TBV_FUSE_GEMM_AR=1`` folds each row-parallel GEMM into its collective (one kernel whose epilogue stores LL
packets into the peers' memory; 5 launches per layer, same bits); it is not the default because it measures
slower (see ``parallel/tp.py``).
All buffers are preallocated so a decode step can be captured in a CUDA graph.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from .. import ops
from ..parallel.tp import TPGroup
from .config import ModelConfig


class LlamaTP:
    def __init__(self, cfg: ModelConfig, tp: TPGroup, weights: Dict[str, torch.Tensor], device, max_tokens: int,
                 max_batch: int, num_blocks: int, block_size: int = 16, max_attn_splits: int = 32):
        cfg.check_tp(tp.world)
        self.cfg, self.tp, self.w, self.device = cfg, tp, weights, torch.device(device)
        self.block_size, self.num_blocks = block_size, num_blocks
        self.nq = cfg.num_heads // tp.world
        self.nkv = cfg.kv_heads_per_rank(tp.world)
        self.D = cfg.head_dim
        self.ipr = cfg.intermediate_size // tp.world
        self.vpr = cfg.vocab_size // tp.world
        self.max_tokens, self.max_batch, self.max_attn_splits = max_tokens, max_batch, max_attn_splits
        bf, dev, H = torch.bfloat16, self.device, cfg.hidden_size
        qkv_dim = (self.nq + 2 * self.nkv) * self.D
        # activations (row-prefix slices of these are what every call uses)
        self.h = torch.zeros(max_tokens, H, dtype=bf, device=dev)        # residual stream
        self.xn = torch.zeros(max_tokens, H, dtype=bf, device=dev)       # normalised input / partial sums
        self.part = torch.zeros(max_tokens, H, dtype=bf, device=dev)     # partial sums / normalised
        self.qkv = torch.zeros(max_tokens, qkv_dim, dtype=bf, device=dev)
        self.attn = torch.zeros(max_tokens, self.nq * self.D, dtype=bf, device=dev)
        self.act = torch.zeros(max_tokens, self.ipr, dtype=bf, device=dev)
        self.gu = None   # [max_tokens, 2 * ipr], allocated on first sequence-parallel prefill
        self.xl = torch.zeros(max_batch, H, dtype=bf, device=dev)        # rows that get logits
        self.logits = torch.zeros(max_batch, self.vpr, dtype=bf, device=dev)
        self.argmax_ws = ops.argmax_workspace(max_batch, dev)
        self.attn_ws = ops.attn_workspace(max_batch, self.nq, self.nkv, max_attn_splits, dev)   # kv splits are a decode-only device
        idx_off, rec = ops.cand_layout(max_batch)
        self.cand = torch.zeros(rec, dtype=torch.uint8, device=dev)
        self.cand_all = torch.zeros(tp.world, rec, dtype=torch.uint8, device=dev)
        self.cos_sin = ops.rope_cos_sin(self.D, cfg.max_position, cfg.rope_theta, dev, cfg.rope_scaling)
        self.scale = 1.0 / math.sqrt(self.D)
        # Decode GEMMs may announce the next GEMM's weights (forward).  Edges: bit 0 qkv -> o_proj, 1 o_proj -> gate_up,
        # 2 gate_up -> down, 3 down -> next layer's qkv (or the LM head).  Measured one edge at a time on the 8B shape: only
        # o_proj -> gate_up pays (-3.0 % of the step at TP=1, -2.0 % at TP=2 shapes); the others are neutral or cost 0.5-1.7 %.
        self.l2_prefetch = 0 if os.environ.get("TBV_L2_PREFETCH", "1") == "0" else int(os.environ.get("TBV_L2_PREFETCH_EDGES", "2"))
        # paged KV cache, one pair per layer: [num_blocks * block_size, nkv, D]
        self.k_cache = [torch.zeros(num_blocks * block_size, self.nkv, self.D, dtype=bf, device=dev) for _ in range(cfg.num_layers)]
        self.v_cache = [torch.zeros(num_blocks * block_size, self.nkv, self.D, dtype=bf, device=dev) for _ in range(cfg.num_layers)]

    # -- one forward pass over T token rows ----------------------------------------------------
    def forward(self, T: int, ids: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor, block_tables: torch.Tensor,
                ctx_lens: torch.Tensor, seq_of_query: Optional[torch.Tensor], logit_rows: Optional[torch.Tensor], n_logits: int,
                out_tokens: torch.Tensor, attn_splits: int = 1, prefill_tiles: Optional[torch.Tensor] = None,
                layer_begin: int = 0, layer_end: Optional[int] = None) -> Optional[torch.Tensor]:
        """ids/positions/slot_mapping/ctx_lens: [T]; logit_rows: int64 [n_logits] rows whose next
        token is wanted (None = all T rows, decode).  Writes greedy tokens to out_tokens[:n_logits].
        ``layer_begin`` / ``layer_end`` run a slice of the model (the state between slices lives in this object's
        static buffers): the embedding and first norm belong to the slice that starts at layer 0, the LM head and
        the sampling to the slice that ends at the last layer; other slices return None."""
        cfg, w, tp = self.cfg, self.w, self.tp
        layer_end = cfg.num_layers if layer_end is None else layer_end
        assert T <= self.max_tokens and n_logits <= self.max_batch and 0 <= layer_begin <= layer_end <= cfg.num_layers
        h, xn, part, qkv, attn, act = self.h[:T], self.xn[:T], self.part[:T], self.qkv[:T], self.attn[:T], self.act[:T]
        q_view = qkv.view(T, self.nq + 2 * self.nkv, self.D)[:, : self.nq]
        attn_view = attn.view(T, self.nq, self.D)

        if layer_begin == 0:
            ops.embedding(ids, w["embed"], vocab_start=tp.rank * self.vpr, out=h)
            tp.all_reduce(h)
            ops.rmsnorm(h, w["layers.0.input_norm"], cfg.rms_eps, out=xn)
        # Decode: every GEMM asks for the NEXT GEMM's weights to be brought into L2 while its own epilogue, the kernel
        # boundary and the attention / all-reduce kernel in between would leave HBM idle (ops.prefetch_next).
        pf = self.l2_prefetch if T <= 64 else 0
        for l in range(layer_begin, layer_end):
            p = f"layers.{l}."
            # qkv projection; RoPE and the KV-cache write happen in its epilogue
            if pf & 1:
                ops.prefetch_next(w[p + "o.weight"])
            ops.gemm_qkv_rope(xn, w[p + "qkv.weight"], qkv, positions, self.cos_sin, slot_mapping, self.k_cache[l], self.v_cache[l],
                              self.nq, self.nkv, bias=w.get(p + "qkv.bias"))
            if prefill_tiles is not None:
                ops.prefill_attention(q_view, self.k_cache[l], self.v_cache[l], block_tables, ctx_lens, seq_of_query, prefill_tiles,
                                      attn_view, self.scale, self.block_size)
            else:
                ops.paged_attention(q_view, self.k_cache[l], self.v_cache[l], block_tables, ctx_lens, attn_view, self.scale,
                                    self.block_size, seq_of_query=seq_of_query, splits=attn_splits, workspace=self.attn_ws)
            if pf & 2:
                ops.prefetch_next(w[p + "gate_up.weight"])
            tp.gemm_all_reduce_add_rmsnorm(attn, w[p + "o.weight"], h, w[p + "post_norm"], cfg.rms_eps, out=part)   # part := norm(h), h += sum
            if pf & 4:
                ops.prefetch_next(w[p + "down.weight"])
            ops.gemm(part, w[p + "gate_up.weight"], out=act, epi=ops.EPI_SILU_MUL)
            nxt = w[f"layers.{l + 1}.input_norm"] if l + 1 < cfg.num_layers else w["norm"]
            if pf & 8:
                ops.prefetch_next(w[f"layers.{l + 1}.qkv.weight"] if l + 1 < cfg.num_layers else w["lm_head"])
            tp.gemm_all_reduce_add_rmsnorm(act, w[p + "down.weight"], h, nxt, cfg.rms_eps, out=xn)                  # xn := norm(h) for the next layer
        if layer_end < cfg.num_layers:
            return None
        if logit_rows is None:
            xl = xn
        else:
            xl = self.xl[:n_logits]
            torch.index_select(xn, 0, logit_rows, out=xl)
        logits = self.logits[:n_logits]
        ops.gemm(xl, w["lm_head"], out=logits)
        return self.sample_greedy(logits, n_logits, out_tokens)

    # -- sequence-parallel prefill --------------------------------------------------------------
    def sp_ok(self, T: int) -> bool:
        """Whether a chunk of T token rows can take the sequence-parallel path."""
        tp, cfg = self.tp, self.cfg
        if tp.world < 2 or tp.comm is None or cfg.qkv_bias or T % (tp.world * 16):
            return False
        rpr, H = T // tp.world, cfg.hidden_size
        bn = next((b for b in (256, 128, 64, 32, 16) if rpr % b == 0), 0)
        return bool(bn) and T * H * 2 <= tp.comm.cap and (rpr // bn) * (H // 128) <= 256

    def forward_sp(self, T: int, ids, positions, slot_mapping, block_tables, ctx_lens, seq_of_query, logit_rows, n_logits, out_tokens,
                   prefill_tiles=None):
        """Prefill with the token dimension sharded between the collectives (Megatron-style
        sequence parallelism): residual stream and norms live on T/tp rows; each column-parallel GEMM
        is all-gather -> GEMM, each row-parallel GEMM is GEMM -> reduce-scatter (+ residual + RMSNorm
        on the local rows), both as fused tcgen05 kernels over peer memory."""
        cfg, w, tp, comm = self.cfg, self.w, self.tp, self.tp.comm
        rpr = T // tp.world
        if self.gu is None:
            self.gu = torch.zeros(self.max_tokens, 2 * self.ipr, dtype=torch.bfloat16, device=self.device)
        h, xn, part = self.h[:rpr], self.xn[:rpr], self.part[:rpr]
        qkv, attn, act, gu = self.qkv[:T], self.attn[:T], self.act[:T], self.gu[:T]
        q_view = qkv.view(T, self.nq + 2 * self.nkv, self.D)[:, : self.nq]
        attn_view = attn.view(T, self.nq, self.D)

        def must(ok, what):
            if not ok:
                raise RuntimeError(f"sequence-parallel prefill: the library declined {what}")
            tp.calls += 1
            tp.launches += 2

        ops.embedding(ids, w["embed"], vocab_start=tp.rank * self.vpr, out=self.part[:T])
        must(comm.reduce_scatter(self.part[:T], h), "reduce_scatter(embedding)")
        ops.rmsnorm(h, w["layers.0.input_norm"], cfg.rms_eps, out=xn)
        for l in range(cfg.num_layers):
            p = f"layers.{l}."
            must(comm.allgather_gemm(xn, w[p + "qkv.weight"], qkv), "allgather_gemm(qkv)")
            ops.rope_kv(qkv, positions, self.cos_sin, slot_mapping, self.k_cache[l], self.v_cache[l], self.nq, self.nkv, self.D)
            if prefill_tiles is not None:
                ops.prefill_attention(q_view, self.k_cache[l], self.v_cache[l], block_tables, ctx_lens, seq_of_query, prefill_tiles,
                                      attn_view, self.scale, self.block_size)
            else:
                ops.paged_attention(q_view, self.k_cache[l], self.v_cache[l], block_tables, ctx_lens, attn_view, self.scale,
                                    self.block_size, seq_of_query=seq_of_query, splits=1)
            must(comm.gemm_reduce_scatter(attn, w[p + "o.weight"], residual=h, gamma=w[p + "post_norm"], eps=cfg.rms_eps, y=part),
                 "gemm_reduce_scatter(o_proj)")
            must(comm.allgather_gemm(part, w[p + "gate_up.weight"], gu), "allgather_gemm(gate_up)")
            ops.silu_mul(gu, out=act, interleaved=True)
            nxt = w[f"layers.{l + 1}.input_norm"] if l + 1 < cfg.num_layers else w["norm"]
            must(comm.gemm_reduce_scatter(act, w[p + "down.weight"], residual=h, gamma=nxt, eps=cfg.rms_eps, y=xn),
                 "gemm_reduce_scatter(down_proj)")
        # the rows that get logits may live on any rank: gather the final normalised rows
        must(comm.all_gather(xn, self.part[:T]), "all_gather(final)")
        xl = self.xl[:n_logits]
        torch.index_select(self.part[:T], 0, logit_rows if logit_rows is not None else torch.arange(T, device=self.device), out=xl)
        logits = self.logits[:n_logits]
        ops.gemm(xl, w["lm_head"], out=logits)
        return self.sample_greedy(logits, n_logits, out_tokens)

    def sample_greedy(self, logits: torch.Tensor, n: int, out_tokens: torch.Tensor) -> torch.Tensor:
        """argmax over the vocab shard, then (TP > 1) an all-gather of the per-rank candidates
        and a merge: largest value wins, lowest token id on ties — every rank gets the same token."""
        tp = self.tp
        idx_off, rec = ops.cand_layout(self.max_batch)
        vals = self.cand[: n * 4].view(torch.float32)
        idx = self.cand[idx_off: idx_off + n * 8].view(torch.int64)
        if tp.world == 1:
            ops.argmax(logits, self.argmax_ws, 0, vals, out_tokens[:n])
            return out_tokens
        ops.argmax(logits, self.argmax_ws, tp.rank * self.vpr, vals, idx)
        tp.all_gather(self.cand, self.cand_all)
        ops.argmax_merge_packed(self.cand_all, tp.world, n, out_tokens[:n], max_batch=self.max_batch)
        return out_tokens
