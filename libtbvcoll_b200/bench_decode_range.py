#!/usr/bin/env python3
"""Decode throughput over a range of batch sizes, and prefill throughput, for one model on N GPUs —
the serving-shape configuration (Llama-3-70B shape at TP=8, batch 1-256, prompt 2048).

One engine is built for the largest batch; for every batch size B the paged cache is laid out for
B sequences of ``--context`` tokens (block tables reserved, cache contents left as they are: a decode
step's work does not depend on the cached values), the decode step is captured as a CUDA graph with
the device-side feedback kernel and timed like ``bench.py`` (CUDA events around K replays, barrier +
synchronize on both sides, max over ranks).  With ``--nccl`` the same engine and weights run a second
time with every collective on torch.distributed (NCCL defaults).  Prefill is timed for
``--prefill-batch`` prompts of ``--context`` tokens, once through the sequence-parallel path
(all-gather -> GEMM, GEMM -> reduce-scatter) and once through the all-reduce path.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        -m libtbvcoll_b200.bench_decode_range --model llama3-70b --batches 1,8,64,256 --context 2048 --nccl
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def timed(replay, steps, warmup, world):
    for _ in range(warmup):
        replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        replay()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def decode_ms(eng, B, ctx, steps, warmup, world):
    eng.bm.release_all()
    for b in range(B):
        eng.bm.reserve(b, ctx + steps + warmup + 8)
    eng.bm.sync_to_device()
    ids = torch.randint(0, eng.cfg.vocab_size, (B,), generator=torch.Generator().manual_seed(B)).tolist()
    eng._load_decode_inputs(B, ids, [ctx] * B)
    eng.step_counter.zero_()
    splits = eng.attn_splits_for(B, ctx + steps + warmup)
    g = eng.capture(B, splits, True)
    torch.cuda.synchronize()
    return timed(g.replay, steps, warmup, world), splits


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--batches", default="1,8,64,256")
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--prefill-batch", type=int, default=8)
    ap.add_argument("--nccl", action="store_true", help="also run the same engine with its collectives on NCCL")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    from libtbvcoll_b200.parallel.tp import TPGroup
    from libtbvcoll_b200.tbvcoll import Comm
    cfg = get_config(args.model)
    batches = [int(b) for b in args.batches.split(",")]
    maxb, ctx, chunk = max(batches + [args.prefill_batch]), args.context, 2048
    comm = None
    if world > 1:
        comm = Comm(rank, world, local, "127.0.0.1", int(os.environ.get("MASTER_PORT", "29500")) + 109, cap_bytes=chunk * cfg.hidden_size * 2)
    tp = TPGroup(rank, world, comm)
    eng = Engine(cfg, tp, device=f"cuda:{local}", seed=0, max_batch=maxb, max_seq_len=ctx + args.steps + args.warmup + 32, prefill_chunk=chunk)
    wbytes = cfg.param_count() * 2 / world
    out = {"model": cfg.name, "tp": world, "context": ctx, "weights_gb_per_rank": round(wbytes / 1e9, 2), "decode": [], "prefill": {}}
    for B in batches:
        ms, splits = decode_ms(eng, B, ctx, args.steps, args.warmup, world)
        kv = B * ctx * cfg.kv_heads_per_rank(world) * cfg.head_dim * 2 * 2 * cfg.num_layers
        row = {"batch": B, "ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1), "attn_splits": splits,
               "launches_per_step": eng.launches_per_step,
               "hbm_roofline_ms": round((wbytes + kv) / 6551.4e6, 3), "frac_of_hbm_roofline": round((wbytes + kv) / 6551.4e6 / ms, 3)}
        out["decode"].append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    # prefill: sequence-parallel path vs all-reduce path, second call of each timed (wall clock with synchronize, max over ranks)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=g).tolist() for _ in range(args.prefill_batch)]
    for name, sp in (("sequence_parallel", True), ("all_reduce", False)):
        eng.sp_prefill = sp
        eng.prefill(prompts, 4)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        eng.prefill(prompts, 4)
        torch.cuda.synchronize()
        t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n = args.prefill_batch * ctx
        flops = 2.0 * (cfg.param_count() - cfg.vocab_size * cfg.hidden_size) * n / world
        out["prefill"][name] = {"tokens": n, "ms": round(float(t) * 1e3, 2), "tokens_per_s": round(n / float(t), 1),
                                "gemm_tflops_per_gpu": round(flops / float(t) / 1e12, 1), "chunks_via_sp": eng.sp_chunks}
        if rank == 0:
            print(json.dumps({name: out["prefill"][name]}), flush=True)
    out["collective_fallbacks_to_nccl"] = tp.fallbacks
    if args.nccl and world > 1:
        eng_n = Engine(cfg, TPGroup(rank, world, None), device=f"cuda:{local}", weights=eng.model.w, max_batch=maxb,
                       max_seq_len=ctx + args.steps + args.warmup + 32, prefill_chunk=chunk)
        out["decode_nccl_same_engine"] = []
        for B in batches:
            ms, _ = decode_ms(eng_n, B, ctx, args.steps, args.warmup, world)
            row = {"batch": B, "ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1)}
            out["decode_nccl_same_engine"].append(row)
            if rank == 0:
                print(json.dumps({"nccl_same_engine": row}), flush=True)
        eng_n.graphs.clear()      # captured NCCL collectives must be gone before the process group is
        del eng_n
    torch.cuda.synchronize()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(out, f, indent=1)
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
