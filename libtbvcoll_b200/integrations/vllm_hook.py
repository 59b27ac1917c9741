"""Drop-in hook on vLLM's tensor-parallel all-reduce.

Same behaviour as the reference's monkey-patch (step3b/vllm_tp_bench.py:77-139): only the
TP group is redirected; world size 1 passes through; the library is initialised lazily on
the first TP call (SPMD: all ranks arrive together) or eagerly with ``eager=True`` so the
slot memory is allocated before vLLM sizes its KV cache (``--tbv-eager``, :129-139); per call
the hook checks dtype / size / contiguity, allocates the out-of-place result with
``torch.empty_like``, and calls the pre-bound C function with the CURRENT stream; anything the
library declines (rc -2, unsupported dtype, over capacity, non-contiguous, other groups) is
counted as a fallback and sent to vLLM's original path (NCCL).

vLLM reaches the collective through two doors — ``GroupCoordinator.all_reduce`` in eager
mode and, under torch.compile, the custom op ``torch.ops.vllm.all_reduce`` which lands in
``GroupCoordinator._all_reduce_out_place`` — so both methods are wrapped.

``install_nccl_timing`` is the reference's ``--time-nccl`` shim (:46-75): it wraps the
original method with a per-call stream synchronise and a log2-size histogram.  It is
invasive by design (the reference measured 138.5 -> 113.5 tok/s with it,
reports/10_tp_custom_allreduce.md:38-45) and is for attribution only.
"""
from __future__ import annotations

import ctypes
import os
import time
from typing import Callable, Dict, Optional

import torch

from .. import tbvcoll

stats: Dict[str, float] = {"calls": 0, "fallbacks": 0, "wrapper_s": 0.0}
nccl_hist: Dict[int, list] = {}
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_state = {"installed": False, "tp_name": None, "raw": None, "cap": 0, "orig": None, "orig_oop": None}


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v else default


def _lazy_init(group) -> None:
    """First TP call on every rank: bring the library up for exactly this group."""
    rank, world = group.rank_in_group, group.world_size
    device = torch.cuda.current_device()
    cap = _env_int("TBV_CAP", 4 << 20)                       # the reference bench's default (vllm_tp_bench.py:35)
    port = _env_int("TBV_PORT", 18996)
    peer = os.environ.get("TBV_PEER", os.environ.get("MASTER_ADDR", "127.0.0.1"))
    tbvcoll.init_n(rank, world, device, peer, port, cap)
    _state["raw"], _state["cap"] = tbvcoll.raw_fn(), tbvcoll.cap()


def _is_tp_group(self) -> bool:
    if _state["tp_name"] is None:
        try:
            from vllm.distributed.parallel_state import get_tp_group
            _state["tp_name"] = get_tp_group().unique_name
        except Exception:
            return False
    return getattr(self, "unique_name", None) == _state["tp_name"]


def _try_tbv(self, input_: torch.Tensor) -> Optional[torch.Tensor]:
    # Only real, materialised CUDA tensors may reach the native call.  vLLM's compilation passes trace
    # all_reduce patterns with FakeTensor / proxy tensors (tensor subclasses whose data_ptr is not a
    # device address); handing such a pointer to a kernel is an illegal memory access.
    if type(input_) is not torch.Tensor or torch.compiler.is_compiling():
        return None
    if not _is_tp_group(self):
        return None
    if _state["raw"] is None:
        _lazy_init(self)
    dt = _DT.get(input_.dtype)
    nb = input_.numel() * input_.element_size()
    if dt is None or nb > _state["cap"] or not input_.is_contiguous() or not input_.is_cuda:
        return None
    if nb == 0:
        return input_
    if input_.data_ptr() == 0:
        return None
    out = torch.empty_like(input_)
    st = torch.cuda.current_stream().cuda_stream             # never cached: vLLM switches streams
    rc = _state["raw"](ctypes.c_void_p(input_.data_ptr()), ctypes.c_void_p(out.data_ptr()), nb, dt, ctypes.c_void_p(st))
    if rc == 0:
        return out
    if rc == -2:
        return None
    raise RuntimeError(f"tbv_ar_allreduce failed rc={rc}")


def _make_patched(orig: Callable) -> Callable:
    def patched(self, input_: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return input_
        if torch.compiler.is_compiling():
            # Under torch.compile vLLM routes through the opaque custom op torch.ops.vllm.all_reduce,
            # which lands in _all_reduce_out_place (wrapped below); nothing here may be traced.
            return orig(self, input_)
        t0 = time.perf_counter()
        out = _try_tbv(self, input_)
        stats["calls"] += 1
        if out is not None:
            stats["wrapper_s"] += time.perf_counter() - t0
            return out
        stats["fallbacks"] += 1
        return orig(self, input_)
    return patched


def install(eager: bool = False, group_coordinator_cls=None) -> None:
    """Patch vLLM.  ``group_coordinator_cls`` lets tests pass a stand-in class."""
    if _state["installed"]:
        return
    if group_coordinator_cls is None:
        from vllm.distributed.parallel_state import GroupCoordinator as group_coordinator_cls
    cls = group_coordinator_cls
    _state["orig"] = cls.all_reduce
    _state["orig_oop"] = getattr(cls, "_all_reduce_out_place", None)
    cls.all_reduce = _make_patched(_state["orig"])
    if _state["orig_oop"] is not None:
        # torch.compile path: torch.ops.vllm.all_reduce -> group._all_reduce_out_place
        orig_oop = _state["orig_oop"]

        def patched_oop(self, input_: torch.Tensor) -> torch.Tensor:
            out = _try_tbv(self, input_)
            if out is not None:
                return out
            return orig_oop(self, input_)
        cls._all_reduce_out_place = patched_oop
    _state["installed"], _state["cls"] = True, cls
    if eager:
        from vllm.distributed.parallel_state import get_tp_group
        _lazy_init(get_tp_group())


def uninstall() -> None:
    if not _state["installed"]:
        return
    cls = _state["cls"]
    cls.all_reduce = _state["orig"]
    if _state["orig_oop"] is not None:
        cls._all_reduce_out_place = _state["orig_oop"]
    _state.update(installed=False, tp_name=None, raw=None)


def install_nccl_timing(group_coordinator_cls=None) -> None:
    """Wrap the ORIGINAL all-reduce with perf_counter + stream synchronise per call."""
    if group_coordinator_cls is None:
        from vllm.distributed.parallel_state import GroupCoordinator as group_coordinator_cls
    cls = group_coordinator_cls
    orig = cls.all_reduce

    def timed(self, input_: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return input_
        torch.cuda.current_stream().synchronize()
        t0 = time.perf_counter()
        out = orig(self, input_)
        torch.cuda.current_stream().synchronize()
        dt = time.perf_counter() - t0
        b = max(0, (input_.numel() * input_.element_size()).bit_length() - 1)
        h = nccl_hist.setdefault(b, [0, 0.0])
        h[0] += 1
        h[1] += dt
        return out
    cls.all_reduce = timed


def summary() -> str:
    c, f = int(stats["calls"]), int(stats["fallbacks"])
    per = stats["wrapper_s"] / max(1, c - f) * 1e6
    s = f"tbvcoll hook: {c} calls, {f} fallbacks to NCCL, {per:.2f} us Python wrapper per call"
    for b in sorted(nccl_hist):
        n, t = nccl_hist[b]
        s += f"\n  nccl 2^{b} B: n={n} mean {t / n * 1e6:.1f} us (with per-call sync)"
    return s
