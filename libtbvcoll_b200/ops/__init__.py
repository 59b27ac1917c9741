"""Python entry points of the hand-written sm_100a operators (``tbv_op_*`` in libtbvcoll.so).

Each function takes torch CUDA tensors, checks shapes, and launches the kernel on the
current stream through ctypes — no torch extension, no Triton, no library GEMM.  The
operators fail loudly when the native library is missing: there is no PyTorch fallback on
a GPU.  ``libtbvcoll_b200.ops.reference`` holds the plain fp32 PyTorch statements of the
same math that the tests compare against.

The reference repository has no operator layer (its model layer is vLLM; its own engine is
described only in reports/11_custom_engine.md:10-20); these operators are what that engine
needs on B200: GEMMs (qkv, gate_up+SiLU, o_proj, down_proj, lm_head), RMSNorm, RoPE + KV
write, paged attention, embedding and greedy argmax.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from ..tbvcoll import load_library

c_vp = ctypes.c_void_p
_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    l = load_library()
    I, F, LL, SZ = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_size_t
    l.tbv_op_gemm.argtypes = [c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, I, I, c_vp]
    l.tbv_op_gemm_error.restype = I
    l.tbv_op_gemm_persist_mode.argtypes = [I]
    l.tbv_op_gemm_persist_mode.restype = None
    l.tbv_op_gemm_streamk_min_bytes.argtypes = [ctypes.c_long]
    l.tbv_op_gemm_streamk_min_bytes.restype = None
    l.tbv_op_gemm_qkv_rope.argtypes = [c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, I, c_vp]
    l.tbv_op_gemm_qkv_rope.restype = I
    l.tbv_op_gemm_config.argtypes = [I, I, I, I, ctypes.POINTER(I), ctypes.POINTER(I), ctypes.POINTER(I)]
    l.tbv_op_rmsnorm.argtypes = [c_vp, c_vp, c_vp, I, I, F, c_vp]
    l.tbv_op_add_rmsnorm.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, I, I, F, c_vp]
    l.tbv_op_rope_kv.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, c_vp]
    l.tbv_op_silu_mul.argtypes = [c_vp, c_vp, I, I, c_vp]
    l.tbv_op_silu_mul_interleaved.argtypes = [c_vp, c_vp, I, I, c_vp]
    l.tbv_op_silu_mul_interleaved.restype = I
    l.tbv_op_embedding.argtypes = [c_vp, c_vp, c_vp, I, I, LL, LL, c_vp]
    l.tbv_op_argmax_workspace.argtypes = [I]
    l.tbv_op_argmax_workspace.restype = SZ
    l.tbv_op_argmax.argtypes = [c_vp, I, I, I, LL, c_vp, c_vp, c_vp, c_vp]
    l.tbv_op_argmax_merge.argtypes = [c_vp, c_vp, I, I, LL, c_vp, c_vp]
    l.tbv_op_decode_advance.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, c_vp, c_vp, I, c_vp]
    l.tbv_op_decode_advance.restype = I
    l.tbv_op_gemm_prefetch_next.argtypes = [c_vp, ctypes.c_size_t]
    l.tbv_op_gemm_prefetch_next.restype = None
    l.tbv_op_copy_async.argtypes = [c_vp, c_vp, ctypes.c_size_t, c_vp]
    l.tbv_op_copy_async.restype = I
    l.tbv_op_prefill_attention.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, I, I, I, F, c_vp]
    l.tbv_op_prefill_attention.restype = I
    l.tbv_op_attn_workspace.argtypes = [I, I, I, I]
    l.tbv_op_attn_workspace.restype = SZ
    l.tbv_op_paged_attention.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, I, I, I, I, F, c_vp]
    for n in ("tbv_op_gemm", "tbv_op_rmsnorm", "tbv_op_add_rmsnorm", "tbv_op_rope_kv", "tbv_op_silu_mul", "tbv_op_embedding",
              "tbv_op_argmax", "tbv_op_argmax_merge", "tbv_op_paged_attention"):
        getattr(l, n).restype = I
    _lib = l
    return l


def _st():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]):
    return c_vp(t.data_ptr()) if t is not None else None


def _chk(rc: int, name: str):
    if rc != 0:
        raise RuntimeError(f"{name} failed rc={rc}")


def gemm_persist_mode(mode: Optional[int]) -> None:
    """Selection of the many-token (persistent) GEMM: 0 never, 1 where it is estimated faster, 2 / 3 force
    its 128- / 256-token tile; None = read ``TBV_GEMM_PERSIST`` again (the library reads it once)."""
    lib().tbv_op_gemm_persist_mode(-1 if mode is None else int(mode))


def gemm_streamk_min_bytes(nbytes: Optional[int]) -> None:
    """Smallest weight matrix (bytes) that takes the evenly-split (stream-K) decode GEMM at up to 64 tokens:
    0 = wherever the shape allows, -1 = never, None = read ``TBV_GEMM_SK_MIN`` again (default: never)."""
    lib().tbv_op_gemm_streamk_min_bytes(-2 if nbytes is None else int(nbytes))


launch_count = 0  # kernels launched through this module (for the bench's gpu_launches claim)


def _count(n=1):
    global launch_count
    launch_count += n


EPI_STORE, EPI_SILU_MUL = 0, 1


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         epi: int = EPI_STORE, splits: int = 0, w_is_constant: bool = True) -> torch.Tensor:
    """out[N, M] = x[N, K] @ w[M, K]^T (+ bias) on tcgen05 tensor cores.  ``epi=EPI_SILU_MUL``:
    ``w`` holds gate/up rows interleaved (row 2i = gate_i, row 2i+1 = up_i) and
    out[N, M/2] = silu(gate) * up.

    ``w`` is treated as a constant (a weight): the kernel starts fetching its tiles before it has
    waited for the kernel launched before it.  Pass ``w_is_constant=False`` when ``w`` was produced
    by the preceding kernel on the stream (a copied or dequantised weight, an activation used as
    ``w``); the fetch then follows the dependency wait."""
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and x.is_cuda and w.is_contiguous()
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.stride(1) == 1
    N, K = x.shape
    M = w.shape[0]
    om = M // 2 if epi == EPI_SILU_MUL else M
    if out is None:
        out = torch.empty((N, om), dtype=torch.bfloat16, device=x.device)
    assert out.shape == (N, om) and out.stride(1) == 1
    _chk(lib().tbv_op_gemm(_p(w), _p(x), _p(out), _p(bias), M, N, K, x.stride(0), out.stride(0), epi | (0 if w_is_constant else 0x100), splits, _st()),
         "tbv_op_gemm")
    _count()
    return out


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                  slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nq: int, nkv: int,
                  bias: Optional[torch.Tensor] = None, splits: int = 0) -> torch.Tensor:
    """qkv[N, (nq+2nkv)*128] = x @ w^T (+ bias) with RoPE applied to the q and k heads and the k, v
    heads written to the paged cache, all in the GEMM epilogue (head_dim 128).  Same bits as
    ``gemm`` followed by ``rope_kv``."""
    N, K = x.shape
    M = w.shape[0]
    assert M == (nq + 2 * nkv) * 128 and qkv.shape == (N, M) and positions.dtype is torch.int32 and cos_sin.shape[1] == 128
    _chk(lib().tbv_op_gemm_qkv_rope(_p(w), _p(x), _p(qkv), _p(bias), M, N, K, x.stride(0), qkv.stride(0), _p(positions), _p(cos_sin),
                                    _p(slot_mapping), _p(k_cache), _p(v_cache), nq, nkv, cos_sin.shape[0], splits, _st()),
         "tbv_op_gemm_qkv_rope")
    _count()
    return qkv


def gemm_config(M: int, N: int, K: int, splits: int = 0):
    bn, sp, stg = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().tbv_op_gemm_config(M, N, K, splits, ctypes.byref(bn), ctypes.byref(sp), ctypes.byref(stg))
    return bn.value, sp.value, stg.value


def gemm_error() -> bool:
    return bool(lib().tbv_op_gemm_error())


def interleave_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up weights -> [2I, K] with row 2i = gate_i, row 2i+1 = up_i (the layout
    the SiLU-mul GEMM epilogue expects)."""
    return torch.stack((gate_w, up_w), dim=1).reshape(-1, gate_w.shape[1]).contiguous()


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    hidden = x.shape[-1]
    tokens = x.numel() // hidden
    out = torch.empty_like(x) if out is None else out
    _chk(lib().tbv_op_rmsnorm(_p(x), _p(gamma), _p(out), tokens, hidden, eps, _st()), "tbv_op_rmsnorm")
    _count()
    return out


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float, residual_out: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None):
    """h = bf16(x + residual); returns (RMSNorm(h) * gamma, h).  Defaults are in place: h over
    ``residual``, the normalised rows over ``x``."""
    hidden = x.shape[-1]
    tokens = x.numel() // hidden
    residual_out = residual if residual_out is None else residual_out
    out = x if out is None else out
    _chk(lib().tbv_op_add_rmsnorm(_p(x), _p(residual), _p(gamma), _p(residual_out), _p(out), tokens, hidden, eps, _st()),
         "tbv_op_add_rmsnorm")
    _count()
    return out, residual_out


def rope_cos_sin(head_dim: int, max_pos: int, theta: float, device, scaling: Optional[dict] = None) -> torch.Tensor:
    """[max_pos, head_dim] fp32 table: cos(0..D/2-1) then sin(0..D/2-1) per position; optional
    Llama-3.1 style frequency scaling (``rope_type == "llama3"``)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wl = 2 * math.pi / inv
        smooth = ((old / wl) - lo) / (hi - lo)
        scaled = torch.where(wl > old / lo, inv / factor, inv)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wl <= old / lo) & (wl >= old / hi)
        inv = torch.where(is_mid, mid, scaled)
    f = torch.outer(torch.arange(max_pos, dtype=torch.float32, device=device), inv)
    return torch.cat((f.cos(), f.sin()), dim=-1).contiguous()


def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, slot_mapping: Optional[torch.Tensor],
            k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nq: int, nkv: int, head_dim: int) -> None:
    """In place: rotate the q and k heads of qkv [T, (nq+2nkv)*D]; write k, v rows into the
    paged cache at slot_mapping (int64; negative = skip)."""
    T = qkv.shape[0]
    assert qkv.is_contiguous() and positions.dtype is torch.int32 and cos_sin.dtype is torch.float32
    assert slot_mapping is None or slot_mapping.dtype is torch.int64
    _chk(lib().tbv_op_rope_kv(_p(qkv), _p(positions), _p(cos_sin), _p(slot_mapping), _p(k_cache), _p(v_cache), T, nq, nkv, head_dim,
                              cos_sin.shape[0], _st()), "tbv_op_rope_kv")
    _count()


def silu_mul(x: torch.Tensor, out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """x: [T, 2I] = [gate | up] (or, ``interleaved``, columns g0 u0 g1 u1 ...) -> silu(gate) * up, [T, I]."""
    T, I2 = x.shape
    out = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device) if out is None else out
    fn = lib().tbv_op_silu_mul_interleaved if interleaved else lib().tbv_op_silu_mul
    _chk(fn(_p(x), _p(out), T, I2 // 2, _st()), "tbv_op_silu_mul")
    _count()
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of a vocab shard; ids outside [vocab_start, vocab_start + rows) give zeros (the
    shards are summed by an all-reduce)."""
    assert ids.dtype is torch.int64
    T, H = ids.numel(), table.shape[1]
    out = torch.empty((T, H), dtype=table.dtype, device=table.device) if out is None else out
    _chk(lib().tbv_op_embedding(_p(ids), _p(table), _p(out), T, H, vocab_start, vocab_start + table.shape[0], _st()), "tbv_op_embedding")
    _count()
    return out


def argmax_workspace(tokens: int, device) -> torch.Tensor:
    return torch.zeros(lib().tbv_op_argmax_workspace(tokens), dtype=torch.uint8, device=device)


def argmax(logits: torch.Tensor, workspace: torch.Tensor, index_offset: int = 0, out_val: Optional[torch.Tensor] = None,
           out_idx: Optional[torch.Tensor] = None):
    """Per row: (max logit as fp32, lowest index holding it + index_offset)."""
    T, V = logits.shape
    out_val = torch.empty(T, dtype=torch.float32, device=logits.device) if out_val is None else out_val
    out_idx = torch.empty(T, dtype=torch.int64, device=logits.device) if out_idx is None else out_idx
    _chk(lib().tbv_op_argmax(_p(logits), T, V, logits.stride(0), index_offset, _p(workspace), _p(out_val), _p(out_idx), _st()),
         "tbv_op_argmax")
    _count()
    return out_val, out_idx


def cand_layout(T: int):
    """Byte layout of one rank's greedy candidates: fp32 values, then int64 indices."""
    idx_off = (T * 4 + 15) // 16 * 16
    return idx_off, idx_off + T * 8


def argmax_merge_packed(gathered: torch.Tensor, world: int, T: int, out: torch.Tensor, max_batch: Optional[int] = None) -> torch.Tensor:
    """gathered: uint8 [world, rec]; each record is laid out by ``cand_layout(max_batch or T)``
    and its first T entries are merged."""
    idx_off, rec = cand_layout(max_batch or T)
    base = gathered.data_ptr()
    _chk(lib().tbv_op_argmax_merge(c_vp(base), c_vp(base + idx_off), world, T, rec, _p(out), _st()), "tbv_op_argmax_merge")
    _count()
    return out


def decode_advance(next_ids, ids, positions, ctx_lens, slot_mapping, block_tables, block_size, history, step_counter) -> None:
    B = ids.shape[0]
    _chk(lib().tbv_op_decode_advance(_p(next_ids), _p(ids), _p(positions), _p(ctx_lens), _p(slot_mapping), _p(block_tables),
                                     block_tables.shape[1], block_size, B, _p(history), _p(step_counter),
                                     history.shape[0] if history is not None else 0, _st()), "tbv_op_decode_advance")
    _count()


def prefetch_next(w: Optional[torch.Tensor]) -> None:
    """Announce the weight matrix of the GEMM that will run AFTER the next ``gemm`` / ``gemm_qkv_rope`` call: the CTAs of
    that next call ask for it (up to TBV_L2_PREFETCH_MB, default 32 MB) to be brought into L2 once their own weight
    tiles are requested, so that HBM keeps streaming through the epilogue, the kernel boundary and whatever small kernel
    runs in between.  Holds for one launch; decode-size kernels only (the many-token kernels ignore it).  ``w`` is read
    by that launch: it must stay allocated until the launch has run (a weight, not a temporary)."""
    if w is not None:
        lib().tbv_op_gemm_prefetch_next(_p(w), w.numel() * w.element_size())


def copy_async(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst <- src (same byte count, both contiguous; pinned host or device memory) as one asynchronous copy on the
    current stream.  Unlike ``Tensor.copy_`` it involves no allocator bookkeeping, so it may be captured in a CUDA graph."""
    nb = src.numel() * src.element_size()
    assert nb == dst.numel() * dst.element_size() and dst.is_contiguous() and src.is_contiguous()
    _chk(lib().tbv_op_copy_async(_p(dst), _p(src), nb, _st()), "tbv_op_copy_async")


def attn_workspace(nq_rows: int, nq_heads: int, nkv: int, max_splits: int, device) -> torch.Tensor:
    return torch.zeros(lib().tbv_op_attn_workspace(nq_rows, nq_heads, nkv, max_splits), dtype=torch.uint8, device=device)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, ctx_lens: torch.Tensor,
                    out: torch.Tensor, scale: float, block_size: int, seq_of_query: Optional[torch.Tensor] = None, splits: int = 1,
                    workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [Nq, nq, D] (a strided view into the qkv buffer is fine), caches [slots, nkv, D],
    block_tables [nseq, max_blocks] int32, ctx_lens [Nq] int32 = keys visible to each query
    row, seq_of_query [Nq] int32 (None = row i is sequence i).  Writes out [Nq, nq, D]."""
    Nq, nq, D = q.shape
    nkv = k_cache.shape[-2]
    assert q.stride(2) == 1 and q.stride(1) == D and out.stride(2) == 1 and out.stride(1) == D
    assert block_tables.dtype is torch.int32 and ctx_lens.dtype is torch.int32
    _chk(lib().tbv_op_paged_attention(_p(q), _p(k_cache), _p(v_cache), _p(block_tables), _p(seq_of_query), _p(ctx_lens), _p(out),
                                      _p(workspace), Nq, nq, nkv, D, q.stride(0), out.stride(0), block_size, block_tables.shape[1],
                                      splits, scale, _st()), "tbv_op_paged_attention")
    _count()
    return out


def prefill_tiles(seq_of_row, group: int) -> torch.Tensor:
    """Segments of at most 64 // group consecutive query rows that belong to one sequence, as the
    int32 [ntiles, 2] (first row, count) list ``prefill_attention`` takes.  ``seq_of_row``: host
    sequence (list / CPU tensor) giving the sequence of every query row, rows grouped by sequence
    in position order."""
    import numpy as np
    qt = max(1, 64 // group)
    seqs = np.asarray(seq_of_row.numpy() if hasattr(seq_of_row, "numpy") else list(seq_of_row), dtype=np.int64)
    n = int(seqs.size)
    if n == 0:
        return torch.zeros(0, 2, dtype=torch.int32)
    run_start = np.concatenate(([0], np.nonzero(seqs[1:] != seqs[:-1])[0] + 1))      # first row of every run of equal sequence ids
    run_len = np.diff(np.concatenate((run_start, [n])))
    per_run = (run_len + qt - 1) // qt                                              # tiles per run
    run_of_tile = np.repeat(np.arange(run_start.size), per_run)
    k = np.arange(int(per_run.sum())) - np.repeat(np.cumsum(per_run) - per_run, per_run)   # tile index inside its run
    first = run_start[run_of_tile] + k * qt
    count = np.minimum(qt, run_len[run_of_tile] - k * qt)
    return torch.from_numpy(np.stack([first, count], axis=1).astype(np.int32))


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, ctx_lens: torch.Tensor,
                      seq_of_query: torch.Tensor, tiles: torch.Tensor, out: torch.Tensor, scale: float, block_size: int) -> torch.Tensor:
    """Causal attention of prompt rows over the paged cache with query tiling on tensor cores: up to
    64 (token, head) rows share every K/V tile.  Same arguments as ``paged_attention`` plus ``tiles``
    (device int32 [ntiles, 2] from ``prefill_tiles``)."""
    Nq, nq, D = q.shape
    nkv = k_cache.shape[-2]
    assert q.stride(2) == 1 and q.stride(1) == D and out.stride(2) == 1 and out.stride(1) == D and tiles.dtype is torch.int32
    _chk(lib().tbv_op_prefill_attention(_p(q), _p(k_cache), _p(v_cache), _p(block_tables), _p(seq_of_query), _p(ctx_lens), _p(tiles),
                                        _p(out), tiles.shape[0], nq, nkv, D, q.stride(0), out.stride(0), block_size,
                                        block_tables.shape[1], scale, _st()), "tbv_op_prefill_attention")
    _count()
    return out
