#!/usr/bin/env python3
"""Operator microbenchmarks against the measured roofline (1 GPU).

For every GEMM shape of a decode step (per-rank shapes of a Llama-shaped model at a given
TP degree and batch) this times the tcgen05 kernel on COLD weights: `nbuf` distinct weight
buffers (> L2 in total) are cycled inside one CUDA graph, device time by CUDA events.
Reports achieved HBM GB/s (weights + activations + output bytes) and TFLOP/s as fractions of
MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16), and the same for torch.matmul (cuBLAS) as
the library comparison.  Also times paged attention, RMSNorm and RoPE at decode shapes.

    python -m libtbvcoll_b200.bench_ops --model llama3-8b --tp 2 --batch 8 [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except OSError:
        return 6650.0, 1590.0, "fallback"


def time_graph(fn_list, reps=5):
    """fn_list: callables launched in order inside one graph; returns mean us per callable."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fn_list:
            f()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for f in fn_list:
                f()
        for _ in range(3):
            g.replay()
        s.synchronize()
        best = 1e30
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            s.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e3 / len(fn_list))
    torch.cuda.current_stream().wait_stream(s)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--json", default="")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--only", default="", help="comma list of op names to run (default: all)")
    ap.add_argument("--nbuf", type=int, default=0, help="weight buffers to cycle (default: enough to exceed 512 MB)")
    args = ap.parse_args()
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.models.config import get_config
    cfg = get_config(args.model)
    tp, B, dev = args.tp, args.batch, "cuda"
    hbm, tflops, src = peaks()
    D = cfg.head_dim
    nq, nkv = cfg.num_heads // tp, cfg.kv_heads_per_rank(tp)
    shapes = [("qkv", (nq + 2 * nkv) * D, cfg.hidden_size, 0), ("o_proj", cfg.hidden_size, nq * D, 0),
              ("gate_up+silu", 2 * cfg.intermediate_size // tp, cfg.hidden_size, 1), ("down_proj", cfg.hidden_size, cfg.intermediate_size // tp, 0),
              ("lm_head", cfg.vocab_size // tp, cfg.hidden_size, 0)]
    rows = []
    only = set(filter(None, args.only.split(",")))
    for name, M, K, epi in shapes:
        if only and name not in only:
            continue
        wbytes = M * K * 2
        nbuf = args.nbuf or max(2, min(64, math.ceil((512 << 20) / wbytes)))
        ws = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(nbuf)]
        x = torch.randn(B, K, device=dev, dtype=torch.bfloat16)
        out = torch.empty(B, M // 2 if epi else M, device=dev, dtype=torch.bfloat16)
        us = time_graph([(lambda w=w: ops.gemm(x, w, out=out, epi=epi, splits=args.splits)) for w in ws])
        out2 = torch.empty(B, M, device=dev, dtype=torch.bfloat16)
        us_lib = time_graph([(lambda w=w: torch.matmul(x, w.t(), out=out2)) for w in ws])
        byts = wbytes + B * K * 2 + out.numel() * 2
        gbs = byts / us / 1e3
        row = {"op": name, "M": M, "K": K, "N": B, "us": round(us, 2), "GBs": round(gbs, 1), "frac_hbm_" + src: round(gbs / hbm, 3),
               "TFLOPs": round(2 * M * K * B / us / 1e6, 2), "cublas_us": round(us_lib, 2), "config(bn,splits,stages)": ops.gemm_config(M, B, K, args.splits)}
        rows.append(row)
        print(json.dumps(row), flush=True)
        del ws
    if only and "paged_attention" not in only:
        return
    # attention at decode shape
    bs = 16
    nblk = B * math.ceil(args.ctx / bs) + 1
    L = 8
    kcs = [torch.randn(nblk * bs, nkv, D, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    vcs = [torch.randn(nblk * bs, nkv, D, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    bt = (torch.arange(B * math.ceil(args.ctx / bs), dtype=torch.int32, device=dev) + 1).view(B, -1)
    ctx = torch.full((B,), args.ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, nq, D, device=dev, dtype=torch.bfloat16)
    o = torch.empty_like(q)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = 1
    while splits < 8 and B * nkv * splits * 2 <= 2 * sms and args.ctx // (splits * 2) >= 64:
        splits *= 2
    ws_a = ops.attn_workspace(B, nq, nkv, splits, dev)
    us = time_graph([(lambda l=l: ops.paged_attention(q, kcs[l], vcs[l], bt, ctx, o, 0.088, bs, splits=splits, workspace=ws_a)) for l in range(L)])
    byts = B * args.ctx * nkv * D * 2 * 2
    row = {"op": "paged_attention", "batch": B, "ctx": args.ctx, "nq": nq, "nkv": nkv, "splits": splits, "us": round(us, 2),
           "GBs": round(byts / us / 1e3, 1), "frac_hbm_" + src: round(byts / us / 1e3 / hbm, 3)}
    rows.append(row)
    print(json.dumps(row), flush=True)
    H = cfg.hidden_size
    x, r, gm = (torch.randn(B, H, device=dev, dtype=torch.bfloat16) for _ in range(2)), None, torch.ones(H, device=dev, dtype=torch.bfloat16)
    x = list(x)
    us = time_graph([(lambda: ops.add_rmsnorm(x[0], x[1], gm, 1e-5)) for _ in range(16)])
    rows.append({"op": "add_rmsnorm", "tokens": B, "hidden": H, "us": round(us, 2)})
    print(json.dumps(rows[-1]), flush=True)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"model": cfg.name, "tp": tp, "batch": B, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
