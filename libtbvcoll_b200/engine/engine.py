"""Greedy TP decode engine: chunked prefill, paged KV cache, decode steps under CUDA graphs.

Counterpart of the reference's undocumented-in-code engine (``engine.py`` / ``run_engine.py``
in reports/11_custom_engine.md:8-23: TP=1/2 decode, greedy, KV cache) and of the vLLM call
its bench makes (``LLM.generate`` with temperature 0 and ``ignore_eos=True``,
step3b/vllm_tp_bench.py:148-171).  The reference measured 6.3-7.8 ms of CPU dispatch per
step in its engine and 28.5 -> 7.1 us for a graph-captured segment (:61-72) but could not
capture its CPU-driven collective (:74); here the whole step, collectives included, is one
graph.

Two decode loops over the same captured step:
  * host loop  — every step copies the step's inputs (token ids, positions, cache slots,
    context lengths) host -> device from pinned memory and reads the sampled tokens back;
    this is what a serving front-end does and what ``generate`` uses by default;
  * device loop — a small kernel inside the graph feeds the sampled token back and advances
    positions/slots, so K steps replay back to back with no host round trip.
"""
from __future__ import annotations

import contextlib
import math
import os
import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..models.config import ModelConfig
from ..models.llama import LlamaTP
from ..parallel.tp import TPGroup
from ..utils.weights import RandomSource, shard_for_rank
from .kv_cache import BlockManager


def _nvtx(name: str):
    """NVTX range around a phase when TBV_NVTX=1 (the native library marks every collective under the same knob)."""
    if os.environ.get("TBV_NVTX", "0") == "1" and torch.cuda.is_available():
        return torch.cuda.nvtx.range(name)
    return contextlib.nullcontext()


def prefill_rows(prompts: Sequence[Sequence[int]], tables: np.ndarray, block_size: int):
    """Flat per-row arrays over all prompts, rows grouped by sequence in position order:
    (total rows, sequence of row, position, token id, KV-cache slot, is-last-row-of-its-prompt).
    numpy throughout: a 4096-row prefill must not spend milliseconds in Python loops."""
    B = len(prompts)
    lens = np.fromiter((len(p) for p in prompts), dtype=np.int64, count=B)
    total = int(lens.sum())
    seq_all = np.repeat(np.arange(B, dtype=np.int64), lens)
    starts = np.cumsum(lens) - lens
    pos_all = np.arange(total, dtype=np.int64) - np.repeat(starts, lens)
    ids_all = np.concatenate([np.asarray(p, dtype=np.int64) for p in prompts]) if total else np.zeros(0, dtype=np.int64)
    slots_all = tables[seq_all, pos_all // block_size].astype(np.int64) * block_size + pos_all % block_size
    is_last = pos_all == (lens[seq_all] - 1)
    return total, seq_all, pos_all, ids_all, slots_all, is_last


class _GraphChain:
    """Graphs that are always replayed one after the other on the current stream."""

    def __init__(self, graphs):
        self.graphs = list(graphs)

    def replay(self) -> None:
        for g in self.graphs:
            g.replay()


class Engine:
    def __init__(self, cfg: ModelConfig, tp: Optional[TPGroup] = None, device="cuda:0", weights: Optional[Dict[str, torch.Tensor]] = None,
                 source=None, seed: int = 0, max_batch: int = 8, max_seq_len: int = 1024, block_size: int = 16,
                 prefill_chunk: int = 2048, max_attn_splits: int = 32):
        self.cfg = cfg
        self.tp = tp or TPGroup()
        self.device = torch.device(device)
        self.max_batch, self.max_seq_len, self.block_size = max_batch, max_seq_len, block_size
        self.prefill_chunk = prefill_chunk
        if weights is None:
            source = source or RandomSource(cfg, seed=seed, device=self.device)
            weights = shard_for_rank(cfg, source, self.tp.rank, self.tp.world, self.device)
        max_blocks_per_seq = (max_seq_len + block_size - 1) // block_size
        num_blocks = max_batch * max_blocks_per_seq + 1
        self.bm = BlockManager(num_blocks, block_size, max_batch, max_blocks_per_seq, self.device)
        self.model = LlamaTP(cfg, self.tp, weights, self.device, max_tokens=max(prefill_chunk, max_batch), max_batch=max_batch,
                             num_blocks=num_blocks, block_size=block_size, max_attn_splits=max_attn_splits)
        dev, B = self.device, max_batch
        # Static decode inputs (graph-captured addresses): ONE device block and ONE pinned mirror, so that a step's inputs
        # cross PCIe as a single copy:  ids int64[B] | cache slots int64[B] | positions int32[B] | context lengths int32[B]
        self.in_d = torch.zeros(24 * B, dtype=torch.uint8, device=dev)
        self.in_h = torch.zeros(24 * B, dtype=torch.uint8).pin_memory()
        carve = lambda buf: (buf[0:8 * B].view(torch.int64), buf[8 * B:16 * B].view(torch.int64),
                             buf[16 * B:20 * B].view(torch.int32), buf[20 * B:24 * B].view(torch.int32))
        self.ids, self.slots, self.positions, self.ctx = carve(self.in_d)
        self.ids_h, self.slots_h, self.pos_h, self.ctx_h = carve(self.in_h)
        self.ctx.fill_(1)
        self.ctx_h.fill_(1)
        self.out_tokens = torch.zeros(B, dtype=torch.int64, device=dev)
        self.out_h = torch.zeros(B, dtype=torch.int64).pin_memory()
        self.h2d_bytes_per_step, self.d2h_bytes_per_step = 24 * B, 8 * B
        # serving loop: layers in a short first graph of a step (0 = one graph per step, the default: measured 3.327 ms per step
        # with 0, 3.323 / 3.327 / 3.348 with 1 / 2 / 4 head layers on the 8B shape; replaying the graph costs the host 13 us); see capture()
        self.serve_head_layers = int(os.environ.get("TBV_SERVE_HEAD", "0"))
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.history = torch.zeros(max_seq_len, B, dtype=torch.int64, device=dev)
        # Sequence-parallel prefill (GEMM->reduce-scatter, all-gather->GEMM) for chunks whose row count divides evenly.
        # Off by default: measured slower than the all-reduce path, whose GEMMs are the persistent many-token kernel
        # (8 x 512 tokens, 8B shape, TP=2: 62.7 vs 39.9 ms; 16384 tokens, 70B shape, TP=8: 1623 vs 559 ms).  TBV_SP_PREFILL=1
        # or ``engine.sp_prefill = True`` selects it; both paths produce identical tokens.
        self.sp_prefill = os.environ.get("TBV_SP_PREFILL", "0") == "1"
        self.sp_chunks = 0
        # query-tiled tensor-core attention for prompt rows (TBV_PREFILL_ATTN=rows: one CTA per query row)
        self.tiled_prefill_attention = os.environ.get("TBV_PREFILL_ATTN", "tiled") != "rows"
        self._ids_np, self._pos_np = self.ids_h.numpy(), self.pos_h.numpy()
        self._slots_np, self._ctx_np, self._out_np = self.slots_h.numpy(), self.ctx_h.numpy(), self.out_h.numpy()
        self._tables_np = self.bm.tables_host.numpy()
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.launches_per_step = 0
        self.last_stats: Dict[str, float] = {}

    # ---- prefill ----------------------------------------------------------------------------
    def prefill(self, prompts: Sequence[Sequence[int]], reserve_new: int) -> List[int]:
        """Run the prompts through the model in chunks of at most ``prefill_chunk`` token rows
        (a sequence may straddle chunks: attention reads earlier chunks from the cache).
        Returns the first generated token of every sequence."""
        B = len(prompts)
        assert 0 < B <= self.max_batch
        self.bm.release_all()
        for b, p in enumerate(prompts):
            if len(p) + reserve_new > self.max_seq_len:
                raise ValueError("prompt + new tokens exceed max_seq_len")
            self.bm.reserve(b, len(p) + reserve_new)
        self.bm.sync_to_device()
        total, seq_all, pos_all, ids_all, slots_all, is_last = prefill_rows(prompts, self.bm.tables_host.numpy(), self.bm.block_size)
        first = [0] * B
        dev = self.device
        for c0 in range(0, total, self.prefill_chunk):
            c1 = min(total, c0 + self.prefill_chunk)
            T = c1 - c0
            pos = torch.from_numpy(pos_all[c0:c1].astype(np.int32))
            seqof = torch.from_numpy(seq_all[c0:c1].astype(np.int32))
            last_r = np.nonzero(is_last[c0:c1])[0]
            n_log = int(last_r.size)
            out = torch.zeros(max(n_log, 1), dtype=torch.int64, device=dev)
            logit_rows = torch.from_numpy(last_r if n_log else np.zeros(1, dtype=np.int64)).to(dev)
            tiles = ops.prefill_tiles(seqof, self.model.nq // self.model.nkv).to(dev) if self.tiled_prefill_attention else None
            ids_d, slots_d = torch.from_numpy(ids_all[c0:c1]).to(dev), torch.from_numpy(slots_all[c0:c1]).to(dev)
            pos_d, ctx_d, seq_d = pos.to(dev), (pos + 1).to(dev), seqof.to(dev)
            if self.sp_prefill and self.model.sp_ok(T):
                self.model.forward_sp(T, ids_d, pos_d, slots_d, self.bm.tables, ctx_d, seq_d, logit_rows, max(n_log, 1), out, prefill_tiles=tiles)
                self.sp_chunks += 1
            else:
                self.model.forward(T, ids_d, pos_d, slots_d, self.bm.tables, ctx_d, seq_d, logit_rows, max(n_log, 1), out, attn_splits=1,
                                   prefill_tiles=tiles)
            if n_log:
                toks = out[:n_log].tolist()
                for r, t in zip(last_r.tolist(), toks):
                    first[int(seq_all[c0 + r])] = t
        return first

    # ---- decode -------------------------------------------------------------------------------
    def _decode_step(self, B: int, splits: int, advance: bool, layer_begin: int = 0, layer_end: Optional[int] = None) -> None:
        self.model.forward(B, self.ids[:B], self.positions[:B], self.slots[:B], self.bm.tables, self.ctx[:B], None, None, B,
                           self.out_tokens, attn_splits=splits, layer_begin=layer_begin, layer_end=layer_end)
        if advance and (layer_end is None or layer_end == self.cfg.num_layers):
            ops.decode_advance(self.out_tokens[:B], self.ids[:B], self.positions[:B], self.ctx[:B], self.slots[:B], self.bm.tables,
                               self.block_size, self.history, self.step_counter)

    def attn_splits_for(self, B: int, max_ctx: int) -> int:
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # kv splits are the CTAs of one cluster: the largest power of two (<= 8) that keeps the whole
        # grid in one wave (two CTAs per SM) and leaves at least 64 cached tokens per CTA
        s = 1
        while s < 8 and B * self.model.nkv * s * 2 <= 2 * sms and max_ctx // (s * 2) >= 64:
            s *= 2
        return min(s, self.model.max_attn_splits)

    def capture(self, B: int, splits: int, advance: bool, io: bool = False):
        """Capture one decode step (all layers, both collectives per layer, sampling) as a graph.  ``io=True`` is the
        serving form: the step starts with the copy of the packed inputs from pinned memory and ends with the copy of
        the sampled tokens back to pinned memory, so that a step costs the host one graph launch.  With
        ``serve_head_layers`` > 0 it is captured as TWO graphs, a short head (copy in, embedding, the first layers) and
        the rest, so that the launch of the long tail overlaps the head's execution (the host cannot launch a step
        before it has read the previous step's tokens).  The returned object has ``replay()``."""
        key = (B, splits, advance, io)
        if key in self.graphs:
            return self.graphs[key]
        L = self.cfg.num_layers
        head = min(max(0, self.serve_head_layers), L) if io else 0
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        parts = []
        with torch.cuda.stream(s):
            self._decode_step(B, splits, False)      # eager warm-up: idempotent (no advance)
            s.synchronize()
            n0 = ops.launch_count + self.tp.launches
            for lo, hi in ([(0, head), (head, L)] if 0 < head < L else [(0, L)]):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    if io and lo == 0:
                        ops.copy_async(self.in_d, self.in_h)
                    self._decode_step(B, splits, advance, lo, hi)
                    if io and hi == L:
                        ops.copy_async(self.out_h, self.out_tokens)
                parts.append(g)
            self.launches_per_step = ops.launch_count + self.tp.launches - n0
        torch.cuda.current_stream(self.device).wait_stream(s)
        self.graphs[key] = parts[0] if len(parts) == 1 else _GraphChain(parts)
        return self.graphs[key]

    def _load_decode_inputs(self, B: int, tokens, lens) -> None:
        """Stage one step's inputs in pinned memory (vectorised on the numpy views of the pinned
        tensors) and copy them to the device: the fed token of row b sits at position lens[b]."""
        import numpy as np
        pos = np.asarray(lens, dtype=np.int64)[:B]
        self._ids_np[:B] = np.asarray(tokens, dtype=np.int64)[:B]
        self._pos_np[:B] = pos
        self._ctx_np[:B] = pos + 1
        bs = self.block_size
        self._slots_np[:B] = self._tables_np[np.arange(B), pos // bs].astype(np.int64) * bs + pos % bs
        ops.copy_async(self.in_d, self.in_h)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, loop: str = "host", use_graph: bool = True,
                 eos_id: Optional[int] = None) -> List[List[int]]:
        """Greedy generation.  ``loop="host"``: per-step H2D inputs + D2H tokens (serving shape);
        ``loop="device"``: steps chained on the device, tokens read back once at the end.
        EOS is ignored unless ``eos_id`` is given (the reference bench sets ignore_eos)."""
        B = len(prompts)
        t0 = time.perf_counter()
        with _nvtx("tbv.prefill"):
            first = self.prefill(prompts, max_new_tokens)
            torch.cuda.synchronize(self.device)
        t1 = time.perf_counter()
        outs = [[t] for t in first]
        lens = [len(p) for p in prompts]      # tokens already in the cache per row
        steps = max_new_tokens - 1
        if steps <= 0:
            return outs
        splits = self.attn_splits_for(B, max(lens) + max_new_tokens)
        if loop == "device":
            self._load_decode_inputs(B, first, lens)
            self.step_counter.zero_()
            g = self.capture(B, splits, True) if use_graph else None
            for _ in range(steps):
                if g is not None:
                    g.replay()
                else:
                    self._decode_step(B, splits, True)
            torch.cuda.synchronize(self.device)
            hist = self.history.view(-1)[: steps * B].view(steps, B).cpu()   # the kernel logs rows of B tokens
            for b in range(B):
                outs[b].extend(hist[:, b].tolist())
        else:
            # Serving shape: every step copies its inputs from pinned memory to the device and reads the sampled tokens
            # back.  Positions, cache slots and context lengths of all steps are laid out before the loop (they do not
            # depend on what is sampled); a step then costs the host four small array writes, one graph launch (copy in,
            # the step's kernels, copy out) and one stream synchronisation.
            import numpy as np
            g = self.capture(B, splits, False, io=True) if use_graph else None
            cur = np.asarray(first, dtype=np.int64)
            bs = self.block_size
            pos_all = np.asarray(lens, dtype=np.int64)[None, :] + np.arange(steps, dtype=np.int64)[:, None]      # [steps, B]
            slots_all = self._tables_np[np.arange(B)[None, :], pos_all // bs].astype(np.int64) * bs + pos_all % bs
            pos32, ctx32 = pos_all.astype(np.int32), (pos_all + 1).astype(np.int32)
            ids_np, slots_np, pos_np, ctx_np, out_np = self._ids_np, self._slots_np, self._pos_np, self._ctx_np, self._out_np
            done = np.zeros(B, dtype=bool)
            trace = []
            sync = torch.cuda.current_stream(self.device).synchronize
            for i in range(steps):
                ids_np[:B] = cur
                slots_np[:B] = slots_all[i]
                pos_np[:B] = pos32[i]
                ctx_np[:B] = ctx32[i]
                if g is not None:
                    g.replay()
                else:
                    ops.copy_async(self.in_d, self.in_h)
                    self._decode_step(B, splits, False)
                    ops.copy_async(self.out_h, self.out_tokens)
                sync()
                cur = out_np[:B].copy()
                trace.append((cur, done.copy()))
                if eos_id is not None:
                    done |= cur == eos_id
                    if done.all():
                        break
            for tok, was_done in trace:
                for b in range(B):
                    if not was_done[b]:
                        outs[b].append(int(tok[b]))
        t2 = time.perf_counter()
        self.last_stats = {"prefill_s": t1 - t0, "decode_s": t2 - t1, "decode_steps": steps, "batch": B,
                           "decode_tok_s": B * steps / max(t2 - t1, 1e-9), "attn_splits": splits,
                           "launches_per_step": self.launches_per_step}
        if ops.gemm_error():
            raise RuntimeError("a GEMM barrier wait gave up on the device (see the kernel's watchdog)")
        return outs
