"""Drop-in hook on vLLM's tensor-parallel all-reduce.

Same behaviour as the reference's monkey-patch (step3b/vllm_tp_bench.py:77-139): only the
TP group is redirected; world size 1 passes through; the library is initialised lazily on
the first TP call (SPMD: all ranks arrive together) or eagerly, BEFORE the engine exists, with
``install(eager=True)`` so the slot memory is allocated before vLLM sizes its KV cache
(``--tbv-eager``, :129-139); per call the hook checks dtype / size / contiguity, allocates the
out-of-place result with ``torch.empty_like``, and calls the pre-bound C function with the
CURRENT stream; anything the library declines (rc -2, unsupported dtype, over capacity,
non-contiguous, other groups) is counted as a fallback and sent to vLLM's original path.

Which method is wrapped.  Current vLLM reaches the collective through ONE run-time door,
``GroupCoordinator._all_reduce_out_place``: ``all_reduce`` itself only forwards to the custom op
``torch.ops.vllm.all_reduce`` (so that Dynamo can trace it), whose implementation calls that
method.  Where it exists only that method is wrapped — ``all_reduce`` stays untouched, nothing
of the hook is ever traced by torch.compile or by vLLM's pattern-matcher passes, and eager and
compiled mode take the same path.  On a vLLM without it, ``all_reduce`` is wrapped like the
reference does (and steps aside while a compiler is tracing).

The per-call path is flat, like the reference's (:96-114, measured 4.1 us of Python per call,
reports/10_tp_custom_allreduce.md:181-195): the TP group object, the C function, the dtype
table, ``empty_like`` and the raw-stream getter are bound once; a call does one identity
test, one dict lookup, three tensor queries, one allocation and one ctypes call.

``install_nccl_timing`` is the reference's ``--time-nccl`` shim (:46-75): it wraps the
original TP all-reduce (other groups pass through untimed, :52-58) with a per-call stream
synchronise and a log2-size histogram.  It is invasive by design (the reference measured
138.5 -> 113.5 tok/s with it, reports/10_tp_custom_allreduce.md:38-45): attribution only.
"""
from __future__ import annotations

import os
import sys
import time
from typing import Callable, Dict, Optional

import torch

from .. import tbvcoll

stats: Dict[str, float] = {"calls": 0, "fallbacks": 0, "wrapper_s": 0.0}
nccl_hist: Dict[int, list] = {}
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_state = {"installed": False, "cls": None, "door": None, "orig": None, "tp": None, "fast": None, "world": 0, "dead": False}


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v else default


def _raw_stream_getter() -> Callable[[], int]:
    """The current CUDA stream as an integer, read on EVERY call (vLLM switches streams; a cached
    stream was a real race in the reference, reports/10_tp_custom_allreduce.md:415-420).  The
    private raw getter avoids building a Stream object per call; the public API is the fallback."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    try:
        dev = torch.cuda.current_device()
        if raw is not None:
            raw(dev)
            return lambda: raw(dev)
    except Exception:
        pass
    cur = torch.cuda.current_stream
    return lambda: cur().cuda_stream


def _bind_fast() -> None:
    """Bind everything the per-call path needs, once (after the library is up)."""
    raw, cap = tbvcoll.raw_fn(), tbvcoll.cap()
    dtmap, empty_like, stream, tensor_t = dict(_DT), torch.empty_like, _raw_stream_getter(), torch.Tensor

    def fast(input_):
        # Only real, materialised CUDA tensors may reach the native call: tensor subclasses (the fake /
        # proxy tensors of a tracer) have no device address.
        if type(input_) is not tensor_t:
            return None
        dt = dtmap.get(input_.dtype)
        if dt is None:
            return None
        nb = input_.numel() * input_.element_size()
        if nb > cap or not input_.is_cuda or not input_.is_contiguous():
            return None
        if nb == 0:
            return input_
        p = input_.data_ptr()
        if p == 0:
            return None
        out = empty_like(input_)
        rc = raw(p, out.data_ptr(), nb, dt, stream())
        if rc == 0:
            return out
        if rc == -2:
            return None
        raise RuntimeError(f"tbv_ar_allreduce failed rc={rc}")

    _state["fast"] = fast


def _init(rank: int, world: int, device: int) -> None:
    cap = _env_int("TBV_CAP", 4 << 20)                       # the reference bench's default (vllm_tp_bench.py:35)
    port = _env_int("TBV_PORT", 18996)
    peer = os.environ.get("TBV_PEER", os.environ.get("MASTER_ADDR", "127.0.0.1"))
    tbvcoll.init_n(rank, world, device, peer, port, cap)
    _state["world"] = world
    _bind_fast()


def init_from_env() -> None:
    """Bring the library up before any engine exists (the reference's --tbv-eager,
    step3b/vllm_tp_bench.py:129-139): rank, world size and device come from the launcher's
    RANK / WORLD_SIZE / LOCAL_RANK, as with vLLM's external launcher where the TP group is the
    whole world.  Every rank must call this at the same point."""
    if _state["fast"] is not None:
        return
    rank, world = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1)
    local = _env_int("LOCAL_RANK", rank)
    if world < 2:
        return
    torch.cuda.set_device(local)
    _init(rank, world, local)


def _resolve_tp(self) -> bool:
    """First multi-rank call: find the TP group object; bring the library up for it if that has not
    happened yet (lazy init: SPMD, all ranks arrive together)."""
    if _state["tp"] is None:
        try:
            from vllm.distributed.parallel_state import get_tp_group
            _state["tp"] = get_tp_group()
        except Exception:
            return False
    if self is not _state["tp"]:
        return False
    if _state["fast"] is None:
        _init(self.rank_in_group, self.world_size, torch.cuda.current_device())
    elif _state["world"] != self.world_size:
        # brought up eagerly for the launcher's world, but the TP group is something else: stand aside
        print(f"[tbvcoll hook] library is up for {_state['world']} ranks but the TP group has {self.world_size}: hook disabled",
              file=sys.stderr)
        _state["dead"], _state["fast"] = True, None
        return False
    return True


def _make_patched(orig: Callable, guard_tracing: bool) -> Callable:
    st, state, clock = stats, _state, time.perf_counter
    is_compiling = torch.compiler.is_compiling

    def patched(self, input_):
        if self.world_size == 1:
            return input_ if guard_tracing else orig(self, input_)
        if guard_tracing and is_compiling():
            return orig(self, input_)          # this door can be traced: nothing of the hook may be
        if self is not state["tp"] or state["fast"] is None:
            if state["dead"] or not _resolve_tp(self):
                return orig(self, input_)
        t0 = clock()
        out = state["fast"](input_)
        st["calls"] += 1
        if out is not None:
            st["wrapper_s"] += clock() - t0
            return out
        st["fallbacks"] += 1
        return orig(self, input_)
    return patched


def install(eager: bool = False, group_coordinator_cls=None) -> None:
    """Patch vLLM.  ``eager=True`` also brings the library up right now (see ``init_from_env``) and may be
    given on a second call after a plain ``install()``.  ``group_coordinator_cls`` lets tests pass a stand-in."""
    if not _state["installed"]:
        if group_coordinator_cls is None:
            from vllm.distributed.parallel_state import GroupCoordinator as group_coordinator_cls
        cls = group_coordinator_cls
        door = "_all_reduce_out_place" if hasattr(cls, "_all_reduce_out_place") else "all_reduce"
        orig = getattr(cls, door)
        setattr(cls, door, _make_patched(orig, guard_tracing=(door == "all_reduce")))
        _state.update(installed=True, cls=cls, door=door, orig=orig)
    if eager:
        init_from_env()


def uninstall() -> None:
    if not _state["installed"]:
        return
    setattr(_state["cls"], _state["door"], _state["orig"])
    _state.update(installed=False, cls=None, door=None, orig=None, tp=None, fast=None, world=0, dead=False)


def install_nccl_timing(group_coordinator_cls=None) -> None:
    """Wrap the ORIGINAL all-reduce of the TP group with perf_counter + stream synchronise per call;
    every other group passes through untouched (step3b/vllm_tp_bench.py:52-58)."""
    if group_coordinator_cls is None:
        from vllm.distributed.parallel_state import GroupCoordinator as group_coordinator_cls
    cls = group_coordinator_cls
    door = "_all_reduce_out_place" if hasattr(cls, "_all_reduce_out_place") else "all_reduce"
    orig = getattr(cls, door)
    tp = {"obj": None}

    def timed(self, input_):
        if self.world_size == 1:
            return orig(self, input_) if door != "all_reduce" else input_
        if tp["obj"] is None:
            try:
                from vllm.distributed.parallel_state import get_tp_group
                tp["obj"] = get_tp_group()
            except Exception:
                tp["obj"] = False
        if self is not tp["obj"] or torch.compiler.is_compiling():
            return orig(self, input_)
        t0 = time.perf_counter()
        out = orig(self, input_)
        torch.cuda.current_stream().synchronize()     # NCCL only enqueues: wait, to count what the hook's device time counts
        dt = time.perf_counter() - t0
        b = max(0, (input_.numel() * input_.element_size()).bit_length() - 1)
        h = nccl_hist.setdefault(b, [0, 0.0])
        h[0] += 1
        h[1] += dt
        return out
    setattr(cls, door, timed)


def summary() -> str:
    c, f = int(stats["calls"]), int(stats["fallbacks"])
    per = stats["wrapper_s"] / max(1, c - f) * 1e6
    s = (f"tbvcoll hook ({_state['door'] or 'not installed'}): {c} calls, {f} fallbacks to NCCL, {per:.2f} us per hooked call "
         f"(Python wrapper + native enqueue; the native part is the `enq` column of stats5)")
    for b in sorted(nccl_hist):
        n, t = nccl_hist[b]
        s += f"\n  nccl 2^{b} B: n={n} mean {t / n * 1e6:.1f} us (with per-call sync)"
    return s
