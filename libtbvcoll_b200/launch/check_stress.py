#!/usr/bin/env python3
"""Slot-reuse stress on real ranks: thousands of all-reduces issued back to back with no
synchronisation in between, every result verified afterwards.  This is the check that finds
completion-order and slot-recycling races which a per-call synchronise hides (the reference
runs the same kind of test in step4/test_stress.py:17-42).

How it is built here:
  * all inputs of a rank live in ONE [ITERS, n] tensor drawn from a generator seeded with the
    rank, all outputs in another; the calls walk over the rows.  Nothing is allocated inside the
    loop, so the caching allocator cannot alias a buffer that a queued call still reads;
  * every rank rebuilds every other rank's tensor from its seed, and the expected rows are the
    fixed-order (rank 0..N-1) fp32 sum rounded once — no other collective library is the oracle;
  * GAP=mem puts a copy larger than L2 between two calls (a decode step's weight stream),
    GAP=compute a bf16 matmul; GAP=none (default) issues the calls as fast as the host can.
Prints one JSON line per rank and exits non-zero on any mismatch or library error.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m libtbvcoll_b200.launch.check_stress
    env: BYTES (57344)  ITERS (2000)  DT (bf16|f16|f32)  GAP (none|mem|compute)  PORT (18998)  CAP (= BYTES)
"""
import json
import os
import sys

import torch

from libtbvcoll_b200 import tbvcoll

DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def rank_inputs(r: int, iters: int, n: int, dtype, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(77001 + r)
    return torch.randn((iters, n), generator=g, device=device, dtype=torch.float32).mul_(3.0).to(dtype)


def make_gap(kind: str):
    if kind == "mem":
        src = torch.empty(384 << 20, dtype=torch.uint8, device="cuda")      # larger than the 126 MB L2
        dst = torch.empty_like(src)
        return lambda: dst.copy_(src)
    if kind == "compute":
        a = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
        return lambda: torch.matmul(a, a)
    return None


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", "2"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    nbytes, iters = int(os.environ.get("BYTES", "57344")), int(os.environ.get("ITERS", "2000"))
    dtype = DTYPES[os.environ.get("DT", "bf16")]
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tbvcoll.init_n(rank, world, local, os.environ.get("PEER_IP", "127.0.0.1"), int(os.environ.get("PORT", "18998")),
                   int(os.environ.get("CAP", str(nbytes))))
    n = nbytes // torch.empty((), dtype=dtype).element_size()
    mine = rank_inputs(rank, iters, n, dtype, dev)
    outs = torch.zeros_like(mine)
    gap = make_gap(os.environ.get("GAP", "none"))
    torch.cuda.synchronize()

    declined = 0
    for it in range(iters):                     # no synchronisation anywhere in this loop
        if not tbvcoll.all_reduce(mine[it], outs[it]):
            declined += 1
        if gap is not None:
            gap()
    torch.cuda.synchronize()

    # expected rows, rebuilt locally in chunks of iterations to bound memory
    bad_rows, bad_elems, first = 0, 0, None
    step = max(1, (256 << 20) // max(1, n * 4 * world))
    for lo in range(0, iters, step):
        hi = min(iters, lo + step)
        acc = None
        for r in range(world):
            part = (mine if r == rank else rank_inputs(r, iters, n, dtype, dev))[lo:hi].float()
            acc = part if acc is None else acc + part
        wrong = (outs[lo:hi] != acc.to(dtype))
        rows = wrong.any(dim=1)
        if bool(rows.any()):
            bad_rows += int(rows.sum())
            bad_elems += int(wrong.sum())
            if first is None:
                first = lo + int(torch.nonzero(rows)[0])
    pre, xfer, post, enq, drain, ncalls = tbvcoll.stats5()
    rec = {"rank": rank, "world": world, "dtype": str(dtype).replace("torch.", ""), "bytes": nbytes, "iters": iters,
           "gap": os.environ.get("GAP", "none"), "async": tbvcoll.is_async(), "declined": declined, "bad_rows": bad_rows,
           "bad_elements": bad_elems, "first_bad_iter": first, "library_error": tbvcoll.err(), "collectives": ncalls,
           "mean_wait_for_peers_us": round(xfer, 2), "mean_reduce_us": round(post, 2), "mean_enqueue_us": round(enq, 2)}
    print(json.dumps(rec), flush=True)
    tbvcoll.hist()
    ok = bad_rows == 0 and declined == 0 and not rec["library_error"]
    tbvcoll.fini()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
