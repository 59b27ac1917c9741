"""Tensor-parallel collectives as the model sees them.

``TPGroup`` owns a ``tbvcoll.Comm`` and implements the calls a row-parallel layer makes:
all-reduce, all-reduce fused with residual-add + RMSNorm, all-gather, reduce-scatter.
Whenever the library declines a call (returns False: over capacity, unsupported dtype,
non-contiguous) the group falls back to ``torch.distributed`` exactly like the reference's
vLLM hook does (step3b/vllm_tp_bench.py:108-124), and counts it.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops
from ..tbvcoll import Comm


class TPGroup:
    """``comm=None`` with ``world > 1`` sends every collective to ``torch.distributed`` (NCCL on GPUs):
    the same model code then runs on the library this one replaces, which is how the benchmark's
    same-engine NCCL arm is built (the reference's own experiment: one engine, the all-reduce swapped,
    step3b/vllm_tp_bench.py:119-124).  ``local_stand_in=True`` replaces every collective by its local
    arithmetic on this rank's partial result (no communication, wrong values): one GPU can then run
    one rank's shard of a TP=N model to attribute the compute part of a step kernel by kernel."""

    def __init__(self, rank: int = 0, world: int = 1, comm: Optional[Comm] = None, fallback_group=None,
                 fused_norm_max_bytes: int = 1 << 20, local_stand_in: bool = False):
        self.rank, self.world, self.comm = rank, world, comm
        self.fallback_group = fallback_group
        self.fused_norm_max_bytes = fused_norm_max_bytes
        self.local_stand_in = local_stand_in
        # One-kernel GEMM + all-reduce + norm (LL packets from the GEMM epilogue, the last CTAs to finish reduce
        # and normalise; same bits as the two-kernel form).  Off by default: measured 3 us per call slower than
        # GEMM followed by the fused all-reduce + norm kernel (the next kernel's CTAs get their slots later and have
        # half the time to prefetch weights before the call completes).  TBV_FUSE_GEMM_AR=1 selects it.
        self.fuse_gemm = os.environ.get("TBV_FUSE_GEMM_AR", "0") == "1"
        self.calls = 0
        self.fallbacks = 0
        self.launches = 0   # collective kernels launched (for the bench's gpu_launches claim)

    # -- plain collectives ---------------------------------------------------------------
    def _fallback_all_reduce(self, x: torch.Tensor) -> None:
        if self.local_stand_in:
            return
        self.fallbacks += 1
        if self.fallback_group is None and not (torch.distributed.is_available() and torch.distributed.is_initialized()):
            raise RuntimeError("tbvcoll declined the call and no torch.distributed fallback is initialised")
        if x.is_contiguous():
            torch.distributed.all_reduce(x, group=self.fallback_group)
        else:
            # torch.distributed wants dense tensors (NCCL raises, gloo reduces the wrong elements)
            dense = x.contiguous()
            torch.distributed.all_reduce(dense, group=self.fallback_group)
            x.copy_(dense)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """In place SUM."""
        if self.world == 1:
            return x
        self.calls += 1
        if self.comm is not None and self.comm.all_reduce(x):
            self.launches += 1
            return x
        self._fallback_all_reduce(x)
        return x

    def all_gather(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            out.view(-1).copy_(x.view(-1))
            return out
        self.calls += 1
        if self.comm is not None and self.comm.all_gather(x, out):
            self.launches += 1
            return out
        if self.local_stand_in:
            out.view(self.world, -1).copy_(x.reshape(1, -1).expand(self.world, -1))
            return out
        self.fallbacks += 1
        torch.distributed.all_gather_into_tensor(out, x, group=self.fallback_group)
        return out

    def reduce_scatter(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            out.view(-1).copy_(x.view(-1))
            return out
        self.calls += 1
        if self.comm is not None and self.comm.reduce_scatter(x, out):
            self.launches += 1
            return out
        if self.local_stand_in:
            out.view(-1).copy_(x.view(self.world, -1)[self.rank])
            return out
        self.fallbacks += 1
        torch.distributed.reduce_scatter_tensor(out, x, group=self.fallback_group)
        return out

    # -- fused: row-parallel GEMM + all-reduce + residual + RMSNorm in one kernel ---------------
    def gemm_all_reduce_add_rmsnorm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                                    out: torch.Tensor):
        """out := RMSNorm(h) * gamma, residual := h, with h = sum over ranks of (x @ w^T) + residual.
        One kernel (tcgen05 GEMM whose epilogue stores into the peers' slot memory) when the
        library takes the shape, else GEMM followed by ``all_reduce_add_rmsnorm``."""
        if self.world > 1 and self.comm is not None and self.fuse_gemm:
            self.calls += 1
            if self.comm.gemm_all_reduce_rmsnorm(x, w, residual, gamma, eps, out):
                self.launches += 1
                return out, residual
            self.calls -= 1
        ops.gemm(x, w, out=out)
        return self.all_reduce_add_rmsnorm(out, residual, gamma, eps)

    # -- fused: all-reduce + residual + RMSNorm ---------------------------------------------
    def all_reduce_add_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float):
        """x: this rank's partial sums [T, H].  Afterwards ``residual`` holds
        h = bf16(sum_ranks x) + residual and ``x`` holds RMSNorm(h) * gamma.  One kernel when the
        message is small enough for the one-shot fused kernel, else all-reduce + add-norm."""
        if self.world == 1:
            ops.add_rmsnorm(x, residual, gamma, eps)      # counted by the ops module
            return x, residual
        nbytes = x.numel() * x.element_size()
        if self.comm is not None and nbytes <= self.fused_norm_max_bytes:
            self.calls += 1
            if self.comm.all_reduce_rmsnorm(x, residual, gamma, eps):
                self.launches += 1
                return x, residual
            self.calls -= 1
        self.all_reduce(x)
        ops.add_rmsnorm(x, residual, gamma, eps)
        return x, residual
