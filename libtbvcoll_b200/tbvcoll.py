"""tbvcoll — ctypes handle on ``libtbvcoll.so`` (B200 build).

Same module-level functions, argument orders and return contract as the reference's
binding (step4/tbvcoll.py:14-111): ``init`` is idempotent and raises on failure;
``all_reduce`` is SUM, in place when ``out`` is None, returns ``False`` whenever the
library cannot take the call (the caller then falls back to NCCL) and ``True`` for
0-byte tensors; the CUDA stream is looked up on EVERY call (a cached stream was a real
race in the reference, reports/10_tp_custom_allreduce.md:415-420); ``raw_fn`` hands out
the pre-bound C function for hot paths; the ``stats*`` getters read and reset.

What is new: any world size 1/2/4/8 (``init_n`` / ``TBV_WORLD``), a CPU backend
(``devs="cpu"``) whose calls are queued and completed by ``synchronize()``, a fused
all-reduce + residual + RMSNorm, reduce-scatter / all-gather, ``fini()``, and a
``Comm`` class for explicit communicators (several worlds per process, and emulated
worlds on one GPU for tests).

    import tbvcoll
    tbvcoll.init_n(rank, world, device, "127.0.0.1", port=18995, cap_bytes=8 << 20)
    ok = tbvcoll.all_reduce(t)        # False -> fall back to NCCL
"""
from __future__ import annotations

import atexit
import collections
import ctypes
import os
from typing import Optional, Sequence

import torch

from . import _build

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lib = None
_ready = False
_cap = 0
_device = -1

c_dp = ctypes.POINTER(ctypes.c_double)
c_ullp = ctypes.POINTER(ctypes.c_ulonglong)
c_vp = ctypes.c_void_p


def load_library(so: Optional[str] = None) -> ctypes.CDLL:
    """dlopen the native library (building it first if the in-tree object is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    path = so or os.environ.get("TBV_LIB") or str(_build.ensure_built())
    l = ctypes.CDLL(path)
    l.tbv_ar_init.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_size_t]
    l.tbv_ar_init.restype = ctypes.c_int
    l.tbv_ar_init_n.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_size_t]
    l.tbv_ar_init_n.restype = ctypes.c_int
    l.tbv_ar_allreduce.argtypes = [c_vp, c_vp, ctypes.c_size_t, ctypes.c_int, c_vp]
    l.tbv_ar_allreduce.restype = ctypes.c_int
    l.tbv_ar_stats.argtypes = [c_dp, c_ullp]
    l.tbv_ar_stats4.argtypes = [c_dp] * 4 + [c_ullp]
    l.tbv_ar_stats5.argtypes = [c_dp] * 5 + [c_ullp]
    for n in ("tbv_ar_async", "tbv_ar_err", "tbv_ar_cap", "tbv_ar_sync", "tbv_ar_fini"):
        getattr(l, n).restype = ctypes.c_int
    l.tbv_ar_cap64.restype = ctypes.c_size_t
    l.tbv_ar_comm.restype = c_vp
    # explicit communicators
    l.tbv_comm_create.argtypes = [ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_char_p,
                                  ctypes.c_int, ctypes.c_size_t]
    l.tbv_comm_create_local.argtypes = [ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int, ctypes.c_size_t]
    l.tbv_comm_destroy.argtypes = [c_vp]
    l.tbv_comm_allreduce.argtypes = [c_vp, c_vp, c_vp, ctypes.c_size_t, ctypes.c_int, c_vp]
    l.tbv_comm_allreduce_local.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), ctypes.c_size_t, ctypes.c_int, c_vp]
    l.tbv_comm_allreduce_rmsnorm.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, ctypes.c_int, ctypes.c_int, ctypes.c_float, c_vp]
    l.tbv_comm_allreduce_rmsnorm_local.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_vp, ctypes.POINTER(c_vp),
                                                   ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int, ctypes.c_float, c_vp]
    l.tbv_comm_gemm_allreduce_rmsnorm.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_float, c_vp]
    l.tbv_comm_gemm_allreduce_rmsnorm.restype = ctypes.c_int
    l.tbv_comm_gemm_allreduce_rmsnorm_local.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_vp,
                                                        ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int,
                                                        ctypes.c_int, ctypes.c_int, ctypes.c_float, c_vp]
    l.tbv_comm_gemm_allreduce_rmsnorm_local.restype = ctypes.c_int
    PP, I, F = ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_float
    l.tbv_comm_gemm_reduce_scatter.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, I, I, I, I, F, I, c_vp]
    l.tbv_comm_gemm_reduce_scatter_local.argtypes = [c_vp, PP, PP, PP, PP, c_vp, PP, PP, I, I, I, I, F, I, c_vp]
    l.tbv_comm_allgather_gemm.argtypes = [c_vp, c_vp, c_vp, c_vp, I, I, I, I, I, c_vp]
    l.tbv_comm_allgather_gemm_local.argtypes = [c_vp, PP, PP, PP, I, I, I, I, I, c_vp]
    for n in ("tbv_comm_gemm_reduce_scatter", "tbv_comm_gemm_reduce_scatter_local", "tbv_comm_allgather_gemm", "tbv_comm_allgather_gemm_local"):
        getattr(l, n).restype = I
    l.tbv_comm_reduce_scatter.argtypes = [c_vp, c_vp, c_vp, ctypes.c_size_t, ctypes.c_int, c_vp]
    l.tbv_comm_all_gather.argtypes = [c_vp, c_vp, c_vp, ctypes.c_size_t, c_vp]
    l.tbv_comm_sync.argtypes = [c_vp]
    for n in ("tbv_comm_rank", "tbv_comm_world", "tbv_comm_nslot", "tbv_comm_is_async", "tbv_comm_err", "tbv_comm_has_nvls"):
        getattr(l, n).argtypes = [c_vp]
        getattr(l, n).restype = ctypes.c_int
    l.tbv_comm_cap.argtypes = [c_vp]
    l.tbv_comm_cap.restype = ctypes.c_size_t
    l.tbv_comm_set_algo.argtypes = [c_vp, ctypes.c_int]
    l.tbv_comm_set_nchan.argtypes = [c_vp, ctypes.c_int]
    l.tbv_comm_set_wdog.argtypes = [c_vp, ctypes.c_double]
    l.tbv_comm_skip_next.argtypes = [c_vp, ctypes.c_int]
    l.tbv_comm_mute_rank.argtypes = [c_vp, ctypes.c_int, ctypes.c_int]
    l.tbv_comm_mute_rank.restype = ctypes.c_int
    l.tbv_comm_tag_counts.argtypes = [c_vp, c_ullp, c_ullp]
    l.tbv_comm_tag_counts.restype = ctypes.c_int
    l.tbv_comm_ctx.argtypes = [c_vp, c_vp, ctypes.c_size_t]
    l.tbv_comm_stats5.argtypes = [c_vp] + [c_dp] * 5 + [c_ullp]
    l.tbv_comm_rails.argtypes = [c_vp]
    l.tbv_comm_hist.argtypes = [c_vp]
    l.tbv_comm_last_error.argtypes = [c_vp, c_ullp]
    l.tbv_comm_breadcrumbs.argtypes = [c_vp, ctypes.c_int, c_ullp]
    l.tbv_comm_breadcrumbs.restype = ctypes.c_int
    l.tbv_comm_timestamps.argtypes = [c_vp, ctypes.c_int, c_ullp]
    l.tbv_comm_timestamps.restype = ctypes.c_int
    l.tbv_comm_trace.argtypes = [c_vp, ctypes.c_int, c_ullp, ctypes.c_int]
    l.tbv_comm_trace.restype = ctypes.c_int
    for n in ("tbv_comm_create", "tbv_comm_create_local", "tbv_comm_destroy", "tbv_comm_allreduce", "tbv_comm_allreduce_local",
              "tbv_comm_allreduce_rmsnorm", "tbv_comm_allreduce_rmsnorm_local", "tbv_comm_reduce_scatter", "tbv_comm_all_gather",
              "tbv_comm_sync", "tbv_comm_set_algo", "tbv_comm_set_nchan", "tbv_comm_set_wdog", "tbv_comm_skip_next", "tbv_comm_ctx"):
        getattr(l, n).restype = ctypes.c_int
    _lib = l
    return l


def _stream_of(t: torch.Tensor):
    # looked up per call, never cached
    return c_vp(torch.cuda.current_stream(t.device).cuda_stream) if t.is_cuda else None


ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "ll": 4, "ce": 5}


class Comm:
    """An explicit communicator.  ``Comm(rank, world, device, ...)`` joins a world of
    processes; ``Comm.local(world, device)`` emulates ``world`` ranks on one GPU in
    one process (one cooperative launch per collective) for tests."""

    def __init__(self, rank: int, world: int, device: int, peer_ip: str = "127.0.0.1", port: int = 18995,
                 cap_bytes: int = 8 << 20, _handle=None, _local=False):
        l = load_library()
        self._l = l
        self.is_local = _local
        if _handle is not None:
            self._h = _handle
        else:
            h = c_vp()
            rc = l.tbv_comm_create(ctypes.byref(h), rank, world, device, (peer_ip or "").encode(), port, cap_bytes)
            if rc != 0:
                raise RuntimeError(f"tbv_comm_create failed rc={rc}")
            self._h = h
        self.rank = l.tbv_comm_rank(self._h)
        self.world = l.tbv_comm_world(self._h)
        self.cap = l.tbv_comm_cap(self._h)
        self.device = device
        # CPU backend: the progress thread reads the caller's buffers after the call has returned.  At most
        # TBV_MAXSLOT (32) calls are ever queued, so holding the last 40 tensor pairs keeps every buffer of a
        # queued call alive even when the caller passed a temporary.  (On CUDA, stream order does this job.)
        self._keep = collections.deque(maxlen=40) if device < 0 else None

    @classmethod
    def local(cls, world: int, device: int = 0, cap_bytes: int = 8 << 20) -> "Comm":
        l = load_library()
        h = c_vp()
        rc = l.tbv_comm_create_local(ctypes.byref(h), world, device, cap_bytes)
        if rc != 0:
            raise RuntimeError(f"tbv_comm_create_local failed rc={rc}")
        return cls(0, world, device, _handle=h, _local=True)

    # -- collectives -------------------------------------------------------------------
    def _check(self, t: torch.Tensor, out: Optional[torch.Tensor]) -> Optional[int]:
        if type(t) is not torch.Tensor or not t.is_contiguous() or (self.device >= 0) != t.is_cuda:
            return None   # tensor subclasses (fake / proxy tensors of a tracer) have no device address
        if out is not None and (not out.is_contiguous() or out.dtype is not t.dtype or out.device != t.device):
            return None
        return _DT.get(t.dtype)

    def all_reduce(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
        dt = self._check(t, out)
        if dt is None or (out is not None and out.numel() != t.numel()):
            return False
        nb = t.numel() * t.element_size()
        if nb == 0:
            return True
        if nb > self.cap:
            return False
        if self._keep is not None:
            self._keep.append((t, out))
        rc = self._l.tbv_comm_allreduce(self._h, c_vp(t.data_ptr()), c_vp(out.data_ptr()) if out is not None else None,
                                        nb, dt, _stream_of(t))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_allreduce failed rc={rc}")
        return True

    def all_reduce_local(self, ins: Sequence[torch.Tensor], outs: Optional[Sequence[torch.Tensor]] = None) -> bool:
        """Emulated world: one tensor per rank."""
        outs = list(outs) if outs is not None else list(ins)
        n = self.world
        assert len(ins) == n and len(outs) == n
        dt = _DT.get(ins[0].dtype)
        if dt is None:
            return False
        nb = ins[0].numel() * ins[0].element_size()
        ip = (c_vp * n)(*[t.data_ptr() for t in ins])
        op = (c_vp * n)(*[t.data_ptr() for t in outs])
        rc = self._l.tbv_comm_allreduce_local(self._h, ip, op, nb, dt, _stream_of(ins[0]))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_allreduce_local failed rc={rc}")
        return True

    def all_reduce_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                           residual_out: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None) -> bool:
        """h = bf16(sum over ranks of x) + residual; residual_out = h; y = RMSNorm(h) * gamma.
        In place on ``residual`` and ``x`` when the outputs are None.  False -> caller composes
        all_reduce + the plain fused add+norm op."""
        if x.dtype is not torch.bfloat16 or not x.is_cuda or not x.is_contiguous() or not residual.is_contiguous():
            return False
        residual_out = residual if residual_out is None else residual_out
        y = x if y is None else y
        hidden = x.shape[-1]
        tokens = x.numel() // hidden
        rc = self._l.tbv_comm_allreduce_rmsnorm(self._h, c_vp(x.data_ptr()), c_vp(residual.data_ptr()), c_vp(gamma.data_ptr()),
                                                c_vp(residual_out.data_ptr()), c_vp(y.data_ptr()), tokens, hidden, eps, _stream_of(x))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_allreduce_rmsnorm failed rc={rc}")
        return True

    def all_reduce_rmsnorm_local(self, xs, residuals, gamma, eps, residual_outs=None, ys=None) -> bool:
        n = self.world
        residual_outs = residuals if residual_outs is None else residual_outs
        ys = xs if ys is None else ys
        hidden = xs[0].shape[-1]
        tokens = xs[0].numel() // hidden
        arr = lambda ts: (c_vp * n)(*[t.data_ptr() for t in ts])
        rc = self._l.tbv_comm_allreduce_rmsnorm_local(self._h, arr(xs), arr(residuals), c_vp(gamma.data_ptr()), arr(residual_outs),
                                                      arr(ys), tokens, hidden, eps, _stream_of(xs[0]))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_allreduce_rmsnorm_local failed rc={rc}")
        return True

    def gemm_all_reduce_rmsnorm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                                y: torch.Tensor, residual_out: Optional[torch.Tensor] = None) -> bool:
        """ONE kernel for a row-parallel layer and what follows it: h = bf16(sum over ranks of
        bf16(x @ w^T)) + residual -> ``residual_out`` (default: in place over ``residual``),
        RMSNorm(h) * gamma -> ``y``.  x: [T, K/tp] (rows may be strided), w: [H, K/tp].  False ->
        compose gemm + all_reduce_rmsnorm instead (T > 256, shapes the kernel does not take, ...)."""
        if x.dtype is not torch.bfloat16 or not x.is_cuda or x.stride(1) != 1 or not w.is_contiguous():
            return False
        residual_out = residual if residual_out is None else residual_out
        T, K = x.shape
        H = w.shape[0]
        rc = self._l.tbv_comm_gemm_allreduce_rmsnorm(self._h, c_vp(w.data_ptr()), c_vp(x.data_ptr()), c_vp(residual.data_ptr()),
                                                     c_vp(gamma.data_ptr()), c_vp(residual_out.data_ptr()), c_vp(y.data_ptr()), T, H, K,
                                                     x.stride(0), eps, _stream_of(x))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_gemm_allreduce_rmsnorm failed rc={rc}")
        return True

    def gemm_all_reduce_rmsnorm_local(self, xs, ws, residuals, gamma, eps, ys, residual_outs=None) -> bool:
        n = self.world
        residual_outs = residuals if residual_outs is None else residual_outs
        T, K = xs[0].shape
        H = ws[0].shape[0]
        arr = lambda ts: (c_vp * n)(*[t.data_ptr() for t in ts])
        rc = self._l.tbv_comm_gemm_allreduce_rmsnorm_local(self._h, arr(ws), arr(xs), arr(residuals), c_vp(gamma.data_ptr()),
                                                           arr(residual_outs), arr(ys), T, H, K, xs[0].stride(0), eps, _stream_of(xs[0]))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_gemm_allreduce_rmsnorm_local failed rc={rc}")
        return True

    @staticmethod
    def _rc(rc: int, name: str) -> bool:
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"{name} failed rc={rc}")
        return True

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                            gamma: Optional[torch.Tensor] = None, eps: float = 1e-5, y: Optional[torch.Tensor] = None) -> bool:
        """Row-parallel GEMM whose tile epilogues scatter over NVLink, then the owner of each token
        row reduces it.  x: [T, K/tp], w: [H, K/tp].  With ``out`` [T/tp, H]: out = this rank's rows
        of the sum.  With ``residual`` (updated in place), ``gamma`` and ``y``: residual += sum,
        y = RMSNorm(residual) * gamma on the local T/tp rows (sequence-parallel prefill)."""
        T, K = x.shape
        mode = 0 if residual is None else 1
        p = lambda t: c_vp(t.data_ptr()) if t is not None else None
        rc = self._l.tbv_comm_gemm_reduce_scatter(self._h, p(w), p(x), p(out), p(residual), p(gamma), p(residual), p(y), T, w.shape[0], K,
                                                  x.stride(0), eps, mode, _stream_of(x))
        return self._rc(rc, "tbv_comm_gemm_reduce_scatter")

    def gemm_reduce_scatter_local(self, xs, ws, outs=None, residuals=None, gamma=None, eps=1e-5, ys=None) -> bool:
        n = self.world
        T, K = xs[0].shape
        mode = 0 if residuals is None else 1
        arr = lambda ts: (c_vp * n)(*[t.data_ptr() for t in ts]) if ts is not None else (c_vp * n)()
        rc = self._l.tbv_comm_gemm_reduce_scatter_local(self._h, arr(ws), arr(xs), arr(outs), arr(residuals),
                                                        c_vp(gamma.data_ptr()) if gamma is not None else None, arr(residuals), arr(ys),
                                                        T, ws[0].shape[0], K, xs[0].stride(0), eps, mode, _stream_of(xs[0]))
        return self._rc(rc, "tbv_comm_gemm_reduce_scatter_local")

    def allgather_gemm(self, x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> bool:
        """y[world * rows, M] = all_gather(x)[world * rows, K] @ w[M, K]^T.  x: this rank's token rows.
        Remote rows are staged in this GPU's memory and loaded by TMA from there as soon as their
        chunk has arrived; tiles over local rows start immediately."""
        rows, K = x.shape
        rc = self._l.tbv_comm_allgather_gemm(self._h, c_vp(w.data_ptr()), c_vp(x.data_ptr()), c_vp(y.data_ptr()), rows, w.shape[0], K,
                                             x.stride(0), y.stride(0), _stream_of(x))
        return self._rc(rc, "tbv_comm_allgather_gemm")

    def allgather_gemm_local(self, xs, ws, ys) -> bool:
        n = self.world
        rows, K = xs[0].shape
        arr = lambda ts: (c_vp * n)(*[t.data_ptr() for t in ts])
        rc = self._l.tbv_comm_allgather_gemm_local(self._h, arr(ws), arr(xs), arr(ys), rows, ws[0].shape[0], K, xs[0].stride(0),
                                                   ys[0].stride(0), _stream_of(xs[0]))
        return self._rc(rc, "tbv_comm_allgather_gemm_local")

    def reduce_scatter(self, t: torch.Tensor, out: torch.Tensor) -> bool:
        """out = block ``rank`` of the rank-ordered sum of t (t has world * out.numel() elements)."""
        dt = self._check(t, out)
        if dt is None or t.numel() != out.numel() * self.world:
            return False
        nb = out.numel() * out.element_size()
        if self._keep is not None:
            self._keep.append((t, out))
        rc = self._l.tbv_comm_reduce_scatter(self._h, c_vp(t.data_ptr()), c_vp(out.data_ptr()), nb, dt, _stream_of(t))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_reduce_scatter failed rc={rc}")
        return True

    def all_gather(self, t: torch.Tensor, out: torch.Tensor) -> bool:
        """out[r] = rank r's t."""
        # any dtype can be gathered (bytes are copied), but only real, contiguous tensors on the communicator's side
        if type(t) is not torch.Tensor or type(out) is not torch.Tensor or not t.is_contiguous() or not out.is_contiguous():
            return False
        if (self.device >= 0) != t.is_cuda or out.device != t.device or out.dtype is not t.dtype:
            return False
        if out.numel() * out.element_size() != t.numel() * t.element_size() * self.world:
            return False
        nb = t.numel() * t.element_size()
        if self._keep is not None:
            self._keep.append((t, out))
        rc = self._l.tbv_comm_all_gather(self._h, c_vp(t.data_ptr()), c_vp(out.data_ptr()), nb, _stream_of(t))
        if rc == -2:
            return False
        if rc != 0:
            raise RuntimeError(f"tbv_comm_all_gather failed rc={rc}")
        return True

    # -- control / introspection ---------------------------------------------------------
    def synchronize(self) -> None:
        """CPU backend: wait for every queued call.  CUDA: completion is stream-ordered,
        this only surfaces a sticky error."""
        if self._l.tbv_comm_sync(self._h) != 0:
            raise RuntimeError("tbvcoll: a collective failed (watchdog / peer lost); the communicator is unusable")

    def err(self) -> bool:
        return bool(self._l.tbv_comm_err(self._h))

    def is_async(self) -> bool:
        return bool(self._l.tbv_comm_is_async(self._h))

    def has_nvls(self) -> bool:
        return bool(self._l.tbv_comm_has_nvls(self._h))

    def nslot(self) -> int:
        return self._l.tbv_comm_nslot(self._h)

    def set_algo(self, algo: str) -> None:
        self._l.tbv_comm_set_algo(self._h, ALGOS[algo])

    def set_nchan(self, n: int) -> None:
        self._l.tbv_comm_set_nchan(self._h, n)

    def set_wdog(self, seconds: float) -> None:
        self._l.tbv_comm_set_wdog(self._h, seconds)

    def skip_next(self, n: int = 1) -> None:
        """Host-side fault injection: this rank silently drops its next ``n`` calls."""
        self._l.tbv_comm_skip_next(self._h, n)

    def mute_rank(self, r: int, n: int = 1) -> None:
        """Emulated world, host-side fault injection: emulated rank ``r`` sits out the next ``n``
        collective launches (its CTAs return before pushing), so the others' bounded waits run out."""
        if self._l.tbv_comm_mute_rank(self._h, r, n) != 0:
            raise RuntimeError("tbv_comm_mute_rank: needs an emulated world and a valid rank")

    def tag_counts(self):
        """(checked, bad) sequence stamps since creation (``TBV_TAG=1``; both 0 otherwise)."""
        a, b = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        if self._l.tbv_comm_tag_counts(self._h, ctypes.byref(a), ctypes.byref(b)) != 0:
            raise RuntimeError("tbv_comm_tag_counts failed")
        return a.value, b.value

    def last_error(self):
        a = (ctypes.c_ulonglong * 4)()
        self._l.tbv_comm_last_error(self._h, a)
        return {"code": a[0], "seq": a[1], "where": a[2], "peer": a[3]}

    def breadcrumbs(self, r: int = 0):
        """Device breadcrumbs of (emulated) rank r: 8 integers (see tbv_comm_breadcrumbs)."""
        a = (ctypes.c_ulonglong * 8)()
        if self._l.tbv_comm_breadcrumbs(self._h, r, a) != 0:
            raise RuntimeError("tbv_comm_breadcrumbs failed")
        return list(a)

    def timestamps(self, r: int = 0):
        """%globaltimer stamps (ns) of the last fused GEMM + all-reduce + norm call (see tbv_comm_timestamps)."""
        a = (ctypes.c_ulonglong * 8)()
        if self._l.tbv_comm_timestamps(self._h, r, a) != 0:
            raise RuntimeError("tbv_comm_timestamps failed")
        return list(a)

    def trace(self, r: int = 0, max_rows: int = 1024):
        """Per-call device time stamps still held in the timing ring, oldest first: a list of
        (seq, t_enter, t_pushed, t_ready, t_done) in ns of the GPU's own timer (channel 0, thread 0; a stamp a
        kernel does not take is 0).  The timers of different GPUs are not synchronised: compare differences."""
        a = (ctypes.c_ulonglong * (5 * max_rows))()
        n = self._l.tbv_comm_trace(self._h, r, a, max_rows)
        if n < 0:
            raise RuntimeError("tbv_comm_trace failed")
        return [tuple(a[5 * i:5 * i + 5]) for i in range(n)]

    def stats5(self):
        v = [ctypes.c_double() for _ in range(5)]
        n = ctypes.c_ulonglong()
        self._l.tbv_comm_stats5(self._h, *[ctypes.byref(x) for x in v], ctypes.byref(n))
        return (*[x.value for x in v], n.value)

    def rails(self) -> None:
        self._l.tbv_comm_rails(self._h)

    def hist(self) -> None:
        self._l.tbv_comm_hist(self._h)

    def ctx_blob(self) -> bytes:
        """The device-side context (peer pointers etc.) that fused kernels take by value."""
        buf = ctypes.create_string_buffer(1024)
        if self._l.tbv_comm_ctx(self._h, buf, 1024) != 0:
            raise RuntimeError("tbv_comm_ctx failed")
        return buf.raw

    @property
    def handle(self):
        return self._h

    def destroy(self) -> None:
        if self._h is not None:
            self._l.tbv_comm_destroy(self._h)
            self._h = None


# ---- module-level API with the reference's names ----------------------------------------

def init(rank, devs, peer_ip, port=18995, cap_bytes=8 << 20, so=None):
    """Reference signature (tbvcoll.py:14).  ``devs``: "cpu", "cuda:N"/"N", or any other
    string (e.g. the reference's rail list) meaning the current CUDA device.  World size
    is 2 unless ``TBV_WORLD`` is set."""
    global _ready, _cap, _device
    if _ready:
        return
    l = load_library(so)
    rc = l.tbv_ar_init(rank, (devs or "").encode(), (peer_ip or "").encode(), port, cap_bytes)
    if rc != 0:
        raise RuntimeError(f"tbv_ar_init failed rc={rc}")
    _ready, _cap = True, l.tbv_ar_cap64()
    _device = -1 if (devs or "").startswith("cpu") else 0
    atexit.register(fini)


def init_n(rank, world, device, peer_ip="127.0.0.1", port=18995, cap_bytes=8 << 20, so=None):
    """N-rank bring-up.  ``device`` is a CUDA ordinal, or -1 for the CPU backend."""
    global _ready, _cap, _device
    if _ready:
        return
    l = load_library(so)
    rc = l.tbv_ar_init_n(rank, world, device, (peer_ip or "").encode(), port, cap_bytes)
    if rc != 0:
        raise RuntimeError(f"tbv_ar_init_n failed rc={rc}")
    _ready, _cap, _device = True, l.tbv_ar_cap64(), device
    atexit.register(fini)


def comm() -> Comm:
    """The global communicator wrapped as a ``Comm`` (for the fused/extra collectives)."""
    if not _ready:
        raise RuntimeError("tbvcoll is not initialised")
    return Comm(0, 0, _device, _handle=c_vp(_lib.tbv_ar_comm()))


def all_reduce(t: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
    """SUM over ranks; in place when ``out`` is None.  False = unsupported here, fall back."""
    if not _ready or type(t) is not torch.Tensor or not t.is_contiguous() or (t.is_cuda != (_device >= 0)):
        return False    # tensor subclasses (fake / proxy tensors of a tracer) have no device address
    if out is not None and (not out.is_contiguous() or out.dtype is not t.dtype or out.numel() != t.numel()):
        return False
    dt = _DT.get(t.dtype)
    if dt is None:
        return False
    nb = t.numel() * t.element_size()
    if nb == 0:
        return True
    if nb > _cap:
        return False
    st = c_vp(torch.cuda.current_stream().cuda_stream) if t.is_cuda else None
    rc = _lib.tbv_ar_allreduce(c_vp(t.data_ptr()), c_vp(out.data_ptr()) if out is not None else None, nb, dt, st)
    if rc == -2:
        return False
    if rc != 0:
        raise RuntimeError(f"tbv_ar_allreduce failed rc={rc}")
    return True


def synchronize():
    if _lib.tbv_ar_sync() != 0:
        raise RuntimeError("tbvcoll: a collective failed (watchdog / peer lost)")


def is_async():
    return bool(_lib.tbv_ar_async())


def err():
    return bool(_lib.tbv_ar_err())


def rails():
    """Dump per-peer arrival waits to stderr (and reset)."""
    _lib.tbv_ar_rails()


def hist():
    """Dump the log2-size histogram to stderr (and reset)."""
    _lib.tbv_ar_hist()


def raw_fn():
    """Pre-bound C function ``(in_ptr, out_ptr, nbytes, dtype, stream) -> rc`` for hot
    paths; the caller checks dtype/size/contiguity itself (reference: tbvcoll.py:74-78)."""
    return _lib.tbv_ar_allreduce


def cap():
    return _cap


def stats5():
    """(pre, xfer, post, enq, drain, count) in us; read-and-reset.  On CUDA, xfer and post
    come from device timestamps (kernel entry -> all peers arrived -> done)."""
    v = [ctypes.c_double() for _ in range(5)]
    n = ctypes.c_ulonglong()
    _lib.tbv_ar_stats5(*[ctypes.byref(x) for x in v], ctypes.byref(n))
    return (*[x.value for x in v], n.value)


def stats4():
    pre, xf, post, enq, _, n = stats5()
    return pre, xf, post, enq, n


def stats3():
    pre, xf, post, enq, n = stats4()
    return pre, xf, post, n


def stats():
    a, c = ctypes.c_double(), ctypes.c_ulonglong()
    _lib.tbv_ar_stats(ctypes.byref(a), ctypes.byref(c))
    return a.value, c.value


def fini():
    """Tear the global communicator down (unmap peers, leave the multicast object)."""
    global _ready
    if _ready and _lib is not None:
        _lib.tbv_ar_fini()
    _ready = False
