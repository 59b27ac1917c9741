#!/usr/bin/env python3
"""The collective and fused GEMM + collective kernels in their emulated-ranks form on ONE GPU
(all ranks of a world are CTAs of one launch; ``Comm.local``).  Two uses: a quick device-time
check of a kernel without a multi-GPU box, and a single-process target for Nsight Compute
(ncu must not wrap a multi-rank launch).  Times are CUDA-event times of ``--iters`` launches on
one stream; they are NOT NVLink numbers — peers are regions of the same HBM.

    python -m libtbvcoll_b200.bench_emulated --op ar_rmsnorm_ll --world 8 --tokens 8 --hidden 4096
    ncu --set full --clock-control none -k regex:k_ar_rmsnorm_ll_local -s 3 -c 1 -o prof \
        python -m libtbvcoll_b200.bench_emulated --op ar_rmsnorm_ll --world 8 --iters 6

ops: ar_ll, ar_oneshot, ar_twoshot, ar_rmsnorm (flag form), ar_rmsnorm_ll, gemm_ar_rmsnorm, gemm_rs, ag_gemm
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2048, help="per-rank input features of the GEMM ops")
    ap.add_argument("--m", type=int, default=4096, help="output features of ag_gemm")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from libtbvcoll_b200.tbvcoll import Comm
    W, T, H, K, dev = args.world, args.tokens, args.hidden, args.k, "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, device=dev, generator=g) * s).to(torch.bfloat16)
    cap = max(T * H * 2, (T // max(W, 1)) * max(H, K) * 2, 1 << 16)
    c = Comm.local(W, 0, cap_bytes=cap)
    gamma = torch.ones(H, dtype=torch.bfloat16, device=dev)
    op = args.op
    if op in ("ar_ll", "ar_oneshot", "ar_twoshot"):
        c.set_algo(op[3:])
        ins = [rnd(T * H) for _ in range(W)]
        outs = [torch.empty_like(t) for t in ins]
        call = lambda: c.all_reduce_local(ins, outs)
        nbytes = T * H * 2
    elif op in ("ar_rmsnorm", "ar_rmsnorm_ll"):
        c.set_algo("oneshot" if op == "ar_rmsnorm" else "auto")
        xs, res = [rnd(T, H, s=0.1) for _ in range(W)], [rnd(T, H) for _ in range(W)]
        ro, ys = [torch.empty_like(x) for x in xs], [torch.empty_like(x) for x in xs]
        call = lambda: c.all_reduce_rmsnorm_local(xs, res, gamma, 1e-5, ro, ys)
        nbytes = T * H * 2
    elif op == "gemm_ar_rmsnorm":
        xs, ws = [rnd(T, K) for _ in range(W)], [rnd(H, K, s=0.02) for _ in range(W)]
        res, ys = [rnd(T, H) for _ in range(W)], [torch.empty(T, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
        call = lambda: c.gemm_all_reduce_rmsnorm_local(xs, ws, res, gamma, 1e-5, ys)
        nbytes = H * K * 2
    elif op == "gemm_rs":
        xs, ws = [rnd(T, K) for _ in range(W)], [rnd(H, K, s=0.02) for _ in range(W)]
        res = [rnd(T // W, H) for _ in range(W)]
        ys = [torch.empty(T // W, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
        call = lambda: c.gemm_reduce_scatter_local(xs, ws, residuals=res, gamma=gamma, eps=1e-5, ys=ys)
        nbytes = H * K * 2
    elif op == "ag_gemm":
        M = args.m
        xs, ws = [rnd(T // W, K) for _ in range(W)], [rnd(M, K, s=0.02) for _ in range(W)]
        ys = [torch.empty(T, M, dtype=torch.bfloat16, device=dev) for _ in range(W)]
        call = lambda: c.allgather_gemm_local(xs, ws, ys)
        nbytes = M * K * 2
    else:
        raise SystemExit(f"unknown op {op}")
    assert call(), "the library declined this shape"
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        call()
    e1.record()
    torch.cuda.synchronize()
    assert not c.err()
    print(json.dumps({"op": op, "world": W, "tokens": T, "hidden": H, "k": K, "iters": args.iters,
                      "us_per_call_all_ranks_on_one_gpu": round(e0.elapsed_time(e1) * 1e3 / args.iters, 2),
                      "bytes_per_rank": nbytes}), flush=True)
    c.destroy()


if __name__ == "__main__":
    main()
