#!/usr/bin/env python3
"""All-reduce latency per message size on real ranks, three clocks side by side, with an exact
check of every size — the job of the reference's step4/test_tbvcoll.py (latency table + sanity
check + optional filler work between calls), built on this repository's benchmark helpers.

Per size the table gives
  stream   device time per call of a stream-ordered loop (CUDA events around groups of calls, p50 and
           p99 over the groups, max over ranks) — what a framework that enqueues eagerly sees;
  graph    device time per call when the calls are captured in one CUDA graph (no host launch cost) —
           what a graph-captured decode step sees;
  enqueue  host time spent inside the call (perf_counter around the enqueue loop, nothing waits);
  wait / reduce   the library's own device timestamps: kernel entry -> all peers' data seen -> done;
  verify   the result of seeded random inputs compared bit for bit with the fixed-order fp32 sum.
GAP_US > 0 puts filler work of about that many microseconds between two calls (GAP_MODE=mem: a copy
larger than L2, the weight stream of a decode layer; GAP_MODE=compute: a bf16 matmul), calibrated with
CUDA events; the stream column then shows the latency a call adds on top of the filler.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m libtbvcoll_b200.launch.latency_table
    env: SIZES (4096,57344,229376,1048576)  ITERS (300)  DT (f32|f16|bf16)  GAP_US (0)  GAP_MODE (compute|mem)
         PORT (18995)  PEER_IP  JSON (file to write the rows to)
"""
import json
import os
import statistics
import time

import torch
import torch.distributed as dist

from libtbvcoll_b200 import tbvcoll
from libtbvcoll_b200.bench_allreduce import graph_us

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


class Filler:
    """About `target_us` of device work, made of whole repetitions of one operation."""

    def __init__(self, mode: str, target_us: float):
        self.reps, self.unit_us = 0, 0.0
        if target_us <= 0:
            return
        if mode == "mem":
            src = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
            dst = torch.empty_like(src)
            self.op = lambda: dst.copy_(src)
        else:
            a = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16)
            self.op = lambda: torch.matmul(a, a)
        for _ in range(3):
            self.op()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            self.op()
        e1.record()
        torch.cuda.synchronize()
        self.unit_us = e0.elapsed_time(e1) * 100.0
        self.reps = max(1, round(target_us / self.unit_us))

    def __call__(self):
        for _ in range(self.reps):
            self.op()


def stream_latency(call, filler, iters):
    """p50 / p99 device microseconds per call (minus the filler) and host microseconds per enqueue."""
    group = 10
    n_groups = max(3, iters // group)

    def timed_groups(body):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_groups)]
        host = 0.0
        for a, b in ev:
            a.record()
            for _ in range(group):
                filler()
                t0 = time.perf_counter()
                body()
                host += time.perf_counter() - t0
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) * 1e3 / group for a, b in ev], host / (n_groups * group) * 1e6

    for _ in range(20):
        call()
    torch.cuda.synchronize()
    dist.barrier()
    with_call, enq = timed_groups(call)
    base = statistics.median(timed_groups(lambda: None)[0]) if filler.reps else 0.0
    us = sorted(max(0.0, v - base) for v in with_call)
    t = torch.tensor([statistics.median(us), us[int(0.99 * (len(us) - 1))], enq], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1]), float(t[2])


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", "2"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    iters = int(os.environ.get("ITERS", "300"))
    sizes = [int(x) for x in os.environ.get("SIZES", "4096,57344,229376,1048576").split(",")]
    dtype = DTYPES[os.environ.get("DT", "f32")]
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))      # barriers and max-over-ranks only
    filler = Filler(os.environ.get("GAP_MODE", "compute"), float(os.environ.get("GAP_US", "0")))
    tbvcoll.init_n(rank, world, local, os.environ.get("PEER_IP", "127.0.0.1"), int(os.environ.get("PORT", "18995")), max(sizes))
    es = torch.empty((), dtype=dtype).element_size()
    rows = []
    if rank == 0:
        gap = f"{filler.reps} x {filler.unit_us:.1f} us of {os.environ.get('GAP_MODE', 'compute')}" if filler.reps else "none"
        print(f"# world={world} dtype={str(dtype).replace('torch.', '')} iters={iters} mode={'ASYNC' if tbvcoll.is_async() else 'SYNC'} filler={gap}")
        print("| bytes | stream p50 us | stream p99 us | graph us | enqueue us | wait us | reduce us | algbw GB/s | verify |")
        print("|---|---|---|---|---|---|---|---|---|", flush=True)
    for nb in sizes:
        n = nb // es
        ins = [torch.randn(n, generator=torch.Generator().manual_seed(9100 + r)).to(dtype).cuda() for r in range(world)]
        acc = ins[0].float()
        for t in ins[1:]:
            acc = acc + t.float()
        want, x = acc.to(dtype), ins[rank]
        y = torch.empty_like(x)
        if not tbvcoll.all_reduce(x, y):
            if rank == 0:
                print(f"| {nb} | declined (over capacity or unsupported) | | | | | | | |", flush=True)
            continue
        torch.cuda.synchronize()
        exact = bool(torch.equal(y, want))
        tbvcoll.stats5()                                                       # reset the accumulators
        p50, p99, enq = stream_latency(lambda: tbvcoll.all_reduce(x, y), filler, iters)
        _, wait_us, reduce_us, _, _, _ = tbvcoll.stats5()
        g_us = graph_us(lambda: tbvcoll.all_reduce(x, y), 20, world)
        row = {"bytes": nb, "stream_p50_us": round(p50, 2), "stream_p99_us": round(p99, 2), "graph_us": round(g_us, 2),
               "enqueue_us": round(enq, 2), "wait_us": round(wait_us, 2), "reduce_us": round(reduce_us, 2),
               "algbw_GBs": round(nb / max(p50, 1e-3) / 1e3, 2), "exact": exact}
        rows.append(row)
        if rank == 0:
            print(f"| {nb} | {row['stream_p50_us']} | {row['stream_p99_us']} | {row['graph_us']} | {row['enqueue_us']} | {row['wait_us']} | "
                  f"{row['reduce_us']} | {row['algbw_GBs']} | {'exact' if exact else 'MISMATCH'} |", flush=True)
    if rank == 0 and os.environ.get("JSON"):
        with open(os.environ["JSON"], "w") as f:
            json.dump({"world": world, "dtype": str(dtype), "rows": rows}, f, indent=1)
    tbvcoll.rails()
    bad = any(not r["exact"] for r in rows) or tbvcoll.err()
    tbvcoll.fini()
    dist.destroy_process_group()
    raise SystemExit(1 if bad else 0)


if __name__ == "__main__":
    main()
