#!/usr/bin/env python3
"""Fused row-parallel linear benchmark: X[T, K/tp] x W[H, K/tp]^T, then all-reduce + residual
add + RMSNorm (eps 1e-5, gamma = 1), at TP = the number of ranks launched.

Each form is timed on cold weights (distinct weight buffers cycled inside one CUDA graph,
device time by CUDA events, max over ranks):
  fused    the library's fused form for the size: up to the LL packet limit ONE kernel (tcgen05 GEMM whose
           epilogue stores LL packets into every rank's memory; the last CTAs to finish reduce + norm); above it,
           where the rows divide evenly, the sequence-parallel pair GEMM -> reduce-scatter (tile epilogues
           scatter over NVLink) + residual + norm on T/tp rows, then an all-gather of the normalised rows
  two      this library's GEMM, then its fused all-reduce + residual + RMSNorm kernel (or, above that kernel's
           size limit, all-reduce followed by the add + norm operator)
  stock    torch.matmul (cuBLAS) + torch.distributed.all_reduce (NCCL) + residual add + RMSNorm in
           PyTorch ops — the path the reference's hook replaces (step3b/vllm_tp_bench.py:87-124)
and the roofline of the fused op: the slower of FLOPs / measured GEMM peak, weight+activation
bytes / measured HBM bandwidth, and bytes that must cross NVLink / 770 GB/s per direction.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29551 -m libtbvcoll_b200.bench_fused [--k 14336] [--hidden 4096] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch
import torch.distributed as dist

from .bench_ops import peaks


def time_graph(fns, world, reps=7):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fns:
            f()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for f in fns:
                f()
        for _ in range(3):
            g.replay()
        s.synchronize()
        dist.barrier()
        us = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            s.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3 / len(fns))
    torch.cuda.current_stream().wait_stream(s)
    t = torch.tensor([sorted(us)[len(us) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--k", type=int, default=14336, help="full (unsharded) input features: 14336 = down_proj, 4096 = o_proj")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--tokens", default="1,8,64,256,1024,4096")
    ap.add_argument("--json", default="")
    ap.add_argument("--stamps", action="store_true", help="print the device time stamps of the last one-kernel call of every size")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.tbvcoll import Comm
    H, K = args.hidden, args.k // world
    hbm, tflops, src = peaks()
    toks = [int(t) for t in args.tokens.split(",")]
    comm = Comm(rank, world, local, "127.0.0.1", int(os.environ.get("MASTER_PORT", "29500")) + 107, cap_bytes=max(256, max(toks)) * H * 2)
    nbuf = max(2, min(32, math.ceil((400 << 20) / (H * K * 2))))
    g = torch.Generator(device="cuda").manual_seed(rank)
    ws = [(torch.randn(H, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(nbuf)]
    gamma = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    rows = []
    for T in toks:
        x = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
        res = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        part = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

        rpr = T // world
        h_loc = torch.randn(max(rpr, 1), H, device="cuda", generator=g).to(torch.bfloat16)
        y_loc = torch.empty(max(rpr, 1), H, dtype=torch.bfloat16, device="cuda")
        form = "one kernel (LL packets from the GEMM epilogue)"
        if not comm.gemm_all_reduce_rmsnorm(x, ws[0], res, gamma, 1e-5, y):      # decided from the shape alone: same on every rank
            form = "GEMM->reduce-scatter + norm on T/tp rows, all-gather" if T % (world * 16) == 0 else None

        def fused(w):
            if form and form.startswith("one"):
                assert comm.gemm_all_reduce_rmsnorm(x, w, res, gamma, 1e-5, y)
            else:
                assert comm.gemm_reduce_scatter(x, w, residual=h_loc, gamma=gamma, eps=1e-5, y=y_loc)
                assert comm.all_gather(y_loc, y)

        def two(w):
            ops.gemm(x, w, out=part)
            if not comm.all_reduce_rmsnorm(part, res, gamma, 1e-5):
                assert comm.all_reduce(part)
                ops.add_rmsnorm(part, res, gamma, 1e-5)

        def stock(w):
            p = torch.matmul(x, w.t())
            dist.all_reduce(p)
            h = p + res
            hf = h.float()
            y.copy_(gamma * (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16))

        t_f = time_graph([(lambda w=w: fused(w)) for w in ws], world) if form else float("nan")
        if args.stamps and form and form.startswith("one") and rank == 0:
            ts = comm.timestamps(0)            # of the last call of the graph just replayed
            names = ("first tile resident", "first tile resident", "first finisher starts", "first row pulled", "rows normalised",
                     "last GEMM tile resident", "its accumulator done", "its packets issued")
            print(f"# T={T} stamps (us after the first): " + "; ".join(f"{n} {(v - ts[0]) / 1e3:+.1f}" for n, v in zip(names, ts)), flush=True)
        t_2 = time_graph([(lambda w=w: two(w)) for w in ws], world)
        t_s = time_graph([(lambda w=w: stock(w)) for w in ws], world)
        flops = 2.0 * T * H * K
        mem = (H * K + T * K + 3 * T * H) * 2
        link = (world - 1) * T * H * 2            # bf16 partial tile to every peer
        roof_us = max(flops / (tflops * 1e6), mem / (hbm * 1e3), link / (770.0 * 1e3))
        row = {"tokens": T, "H": H, "K_local": K, "tp": world, "fused_form": form, "fused_us": round(t_f, 2), "two_kernel_us": round(t_2, 2),
               "stock_cublas_nccl_us": round(t_s, 2), "roofline_us": round(roof_us, 2), "fused_frac_of_roofline_" + src: round(roof_us / t_f, 3),
               "fused_over_two_kernel": round(t_2 / t_f, 3), "speedup_vs_stock": round(t_s / t_f, 2)}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"world": world, "rows": rows, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "nvlink_gbs_per_dir": 770, "source": src}}, f, indent=1)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
