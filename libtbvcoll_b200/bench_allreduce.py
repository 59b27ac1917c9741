#!/usr/bin/env python3
"""All-reduce latency / bandwidth sweep: tbvcoll (LL, one-shot, two-shot, NVLS, copy-engine, auto) vs NCCL.

bf16 [tokens, 4096], tokens in {1, 2, 4, ..., 8192} (8 KB - 64 MB), values N(0,1); every
result of this library is checked bit for bit against a fixed-order fp32 oracle before it is
timed.  Timing is stream-ordered like the reference's microbenchmark ("stream-ordered" mode of
step4/allreduce2.cpp:188-200 and step4/test_tbvcoll.py:52-63): calls are issued back to back
without host synchronisation, device time is taken with CUDA events around groups of calls,
the p50 over groups is reported, and the maximum over ranks is what counts.  NCCL runs at its
default settings (NVLink SHARP / NVLS reduction in the switch included where NCCL chooses it).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 -m libtbvcoll_b200.bench_allreduce [--max-tokens 8192] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def p50_us(fn, inner, groups, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)]
    for a, b in ev:
        a.record()
        for _ in range(inner):
            fn()
        b.record()
    torch.cuda.synchronize()
    us = [a.elapsed_time(b) * 1e3 / inner for a, b in ev]
    t = torch.tensor([statistics.median(us), sorted(us)[int(0.99 * (len(us) - 1))]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1])


def graph_us(fn, inner, world):
    """Device-only latency: `inner` calls captured in one CUDA graph (no host launch cost
    between them), best-of-median over replays, max over ranks."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(inner):
                fn()
        g.replay()
        s.synchronize()
        dist.barrier()
        us = []
        for _ in range(15):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            s.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3 / inner)
    torch.cuda.current_stream().wait_stream(s)
    t = torch.tensor([statistics.median(us)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def phase_stats(every: torch.Tensor):
    """The arithmetic of ``trace_breakdown``: ``every`` is int64 [ranks, calls, 5] of (seq, t_enter, t_pushed, t_ready, t_done)
    in ns, each rank's stamps from its own timer.  Returns the per-phase means in us, or None when the ranks hold different calls."""
    n = every.shape[1]
    if n < 2 or not bool((every[:, :, 0] == every[0:1, :, 0]).all()):
        return None                                   # ranks hold different calls: nothing to align
    t = every.double() * 1e-3
    enter, pushed, ready, done = t[:, :, 1], t[:, :, 2], t[:, :, 3], t[:, :, 4]
    gap = enter[:, 1:] - done[:, :-1]                 # end of one call to the entry of the next, same rank
    period = done[:, 1:] - done[:, :-1]
    stamped = (every[:, :, 2] > 0).all(dim=0)         # calls whose kernel stamps the end of its push (on every rank)
    r2 = lambda v: round(float(v), 2)
    out = {"calls": n, "calls_with_push_stamp": int(stamped.sum()),
           "enter_to_all_sources_seen": r2((ready - enter).mean()),
           "reduce_store_done": r2((done - ready).mean()),
           "gap_to_next_call_median": r2(gap.median()), "gap_to_next_call_p90": r2(gap.flatten().quantile(0.9)),
           "period_median": r2(period.median())}
    if bool(stamped.any()):
        wait = (ready - pushed)[:, stamped]
        out.update({"push_issue": r2((pushed - enter)[:, stamped].mean()),
                    "wait_after_push_least_waiting_rank": r2(wait.min(dim=0).values.mean()),
                    "wait_after_push_mean_rank": r2(wait.mean()),
                    "wait_after_push_most_waiting_rank": r2(wait.max(dim=0).values.mean())})
    return out


def trace_breakdown(comm, calls=256):
    """Where the device time of the last `calls` collectives went, from every rank's own time stamps
    (Comm.trace: kernel entry, own payload issued, every source's payload seen, kernel done; channel 0).
    The GPUs' timers are not synchronised, so only differences taken on one rank are used; ranks are then
    compared call by call.  The rank that waited least after its own push was the last to push: its wait is
    the flight + poll time of the exchange, and the spread between ranks is their arrival skew.  All in us."""
    rows = comm.trace(0, 1024)[-calls:]
    n = torch.tensor([len(rows)], dtype=torch.int64, device="cuda")
    dist.all_reduce(n, op=dist.ReduceOp.MIN)
    n = int(n)
    if n < 2:
        return None
    mine = torch.tensor(rows[-n:], dtype=torch.int64, device="cuda")
    world = dist.get_world_size()
    every = torch.empty((world, n, 5), dtype=torch.int64, device="cuda")
    dist.all_gather_into_tensor(every, mine)
    return phase_stats(every)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-tokens", type=int, default=8192)
    ap.add_argument("--min-tokens", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--json", default="")
    ap.add_argument("--algos", default="auto,ll,oneshot,twoshot,nvls")
    ap.add_argument("--trace", action="store_true", help="add the per-phase device-time breakdown of the graph-replayed calls to every row")
    ap.add_argument("--no-nccl", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from libtbvcoll_b200.tbvcoll import Comm
    cap = args.max_tokens * args.hidden * 2
    port = int(os.environ.get("MASTER_PORT", "29500")) + 103
    comm = Comm(rank, world, local, "127.0.0.1", port, cap_bytes=cap)
    algos = [a for a in args.algos.split(",") if (a != "nvls" or comm.has_nvls()) and (a != "ce" or os.environ.get("TBV_CE") == "1")]
    rows = []
    tokens = max(1, args.min_tokens)
    while tokens <= args.max_tokens:
        n = tokens * args.hidden
        nbytes = n * 2
        g = torch.Generator(device="cpu").manual_seed(1000 + rank)
        x = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
        allx = []
        for r in range(world):
            gr = torch.Generator(device="cpu").manual_seed(1000 + r)
            allx.append(torch.randn(n, generator=gr).to(torch.bfloat16).cuda())
        acc = allx[0].float()
        for t in allx[1:]:
            acc = acc + t.float()
        want = acc.to(torch.bfloat16)
        del allx, acc
        out = torch.empty_like(x)
        inner = 20 if nbytes <= (1 << 20) else 5
        groups = 40 if nbytes <= (4 << 20) else 12
        row = {"tokens": tokens, "bytes": nbytes}
        for algo in algos:
            if algo == "ce" and nbytes < (1 << 20):
                continue            # the copy-engine path is a large-message candidate only
            comm.set_algo(algo)
            assert comm.all_reduce(x, out)
            torch.cuda.synchronize()
            exact = bool(torch.equal(out, want))
            if algo != "nvls":
                assert exact, f"{algo} not bit-exact at {nbytes} bytes"
            p50, p99 = p50_us(lambda: comm.all_reduce(x, out), inner, groups, world)
            row[algo] = {"p50_us": round(p50, 2), "p99_us": round(p99, 2), "graph_us": round(graph_us(lambda: comm.all_reduce(x, out), inner, world), 2),
                         "exact_vs_fixed_order_oracle": exact,
                         "busbw_GBs": round(2 * (world - 1) / world * nbytes / p50 / 1e3, 1)}
            if args.trace:
                row[algo]["phases_us"] = trace_breakdown(comm, calls=10 * inner)   # the last replays of the graph
        if args.no_nccl:
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            tokens *= 2
            continue
        y = x.clone()
        p50, p99 = p50_us(lambda: dist.all_reduce(y), inner, groups, world)
        row["nccl"] = {"p50_us": round(p50, 2), "p99_us": round(p99, 2), "graph_us": round(graph_us(lambda: dist.all_reduce(y), inner, world), 2), "busbw_GBs": round(2 * (world - 1) / world * nbytes / p50 / 1e3, 1)}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        tokens *= 2
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"world": world, "dtype": "bf16", "hidden": args.hidden, "nvls": comm.has_nvls(), "rows": rows}, f, indent=1)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
