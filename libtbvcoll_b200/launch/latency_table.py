#!/usr/bin/env python3
"""End-to-end latency table per message size with a sanity check — the role of the reference's
step4/test_tbvcoll.py:12-72: total us per call (host enqueue + device), enqueue cost, the
library's own transfer / post split (device timestamps), algorithm bandwidth, and verify=OK when
a tensor filled with rank+1 sums to world*(world+1)/2.  GAP_US / GAP_MODE (compute|mem) put a
synthetic layer's worth of work between calls, as in the reference.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m libtbvcoll_b200.launch.latency_table
    env: SIZES (4096,57344,229376,1048576) ITERS (300) DT (f32) GAP_US (0) GAP_MODE PORT (18995)
"""
import os
import time

import torch

from libtbvcoll_b200 import tbvcoll


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", "2"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    iters = int(os.environ.get("ITERS", "300"))
    sizes = [int(x) for x in os.environ.get("SIZES", "4096,57344,229376,1048576").split(",")]
    dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[os.environ.get("DT", "f32")]
    gap_us, gap_mode = float(os.environ.get("GAP_US", "0")), os.environ.get("GAP_MODE", "compute")
    torch.cuda.set_device(local)
    reps, one_op = 0, None
    if gap_us > 0:
        if gap_mode == "mem":
            w = torch.randn(64 * 1024 * 1024 // 2, device="cuda", dtype=torch.float16)
            one_op = lambda: w.sum()
        else:
            a = torch.randn(2048, 2048, device="cuda", dtype=torch.float16)
            one_op = lambda: a @ a
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(20):
            one_op()
        torch.cuda.synchronize()
        per = (time.perf_counter() - t0) / 20 * 1e6
        reps = max(1, round(gap_us / per))
        if rank == 0:
            print(f"# GAP {gap_us:.0f}us = {gap_mode} {per:.1f}us x {reps}", flush=True)
    tbvcoll.init_n(rank, world, local, os.environ.get("PEER_IP", "127.0.0.1"), int(os.environ.get("PORT", "18995")), max(sizes))
    if rank == 0:
        print(f"# dtype={dtype} world={world} iters={iters} mode={'ASYNC' if tbvcoll.is_async() else 'SYNC'}")
        print(f"# {'bytes':>9} {'total_us':>9} {'enqueue':>9} {'xfer_us':>8} {'post_us':>8} {'algbw GB/s':>10} {'verify':>7}", flush=True)
    want = world * (world + 1) / 2
    for nb in sizes:
        numel = nb // torch.tensor([], dtype=dtype).element_size()
        t = torch.full((numel,), float(rank + 1), dtype=dtype, device="cuda")
        for _ in range(30):
            for _ in range(reps):
                one_op()
            assert tbvcoll.all_reduce(t), f"{nb} unsupported"
            t.fill_(float(rank + 1))
        torch.cuda.synchronize()
        tbvcoll.stats4()
        t0 = time.perf_counter()
        for _ in range(iters):
            for _ in range(reps):
                one_op()
            tbvcoll.all_reduce(t)
        torch.cuda.synchronize()
        tot = (time.perf_counter() - t0) / iters
        pre, xfer, post, enq, _ = tbvcoll.stats4()
        c = torch.full((numel,), float(rank + 1), dtype=dtype, device="cuda")
        tbvcoll.all_reduce(c)
        torch.cuda.synchronize()
        ok = bool(torch.allclose(c, torch.full_like(c, want), rtol=1e-2, atol=1e-2))
        if rank == 0:
            print(f"  {nb:>9d} {tot * 1e6:>9.1f} {enq:>9.1f} {xfer:>8.1f} {post:>8.1f} {nb / tot / 1e9:>10.2f} {'OK' if ok else 'BAD':>7}", flush=True)
    tbvcoll.rails()
    tbvcoll.fini()


if __name__ == "__main__":
    main()
