#!/usr/bin/env python3
"""Back-to-back calls with no synchronisation between them, everything verified afterwards — the
role of the reference's step4/test_stress.py:17-42 (slot reuse / completion-order races that a
per-call sync hides).  Input of iteration `it` on rank `r` comes from seed it*world + r, so every
rank can rebuild the expected sums locally.  GAP=mem interleaves a 256 MiB reduction between
calls (weight-streaming imitation), as in the reference.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m libtbvcoll_b200.launch.check_stress
    env: BYTES (57344) ITERS (2000) DT (bf16|f16|f32) GAP (none|mem) PORT (18998) CAP
"""
import os

import torch

from libtbvcoll_b200 import tbvcoll


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", "2"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    nb, iters = int(os.environ.get("BYTES", "57344")), int(os.environ.get("ITERS", "2000"))
    gap = os.environ.get("GAP", "none")
    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[os.environ.get("DT", "bf16")]
    torch.cuda.set_device(local)
    tbvcoll.init_n(rank, world, local, os.environ.get("PEER_IP", "127.0.0.1"), int(os.environ.get("PORT", "18998")),
                   int(os.environ.get("CAP", str(nb))))
    numel = nb // torch.tensor([], dtype=dt).element_size()

    def gen(it, r):
        g = torch.Generator(device="cuda").manual_seed(it * world + r)
        return ((torch.rand(numel, generator=g, device="cuda") - 0.5) * 10).to(dt)

    filler = torch.randn(256 * 1024 * 1024 // 2, device="cuda", dtype=torch.float16) if gap == "mem" else None
    outs, ins = [], []
    for it in range(iters):
        x = gen(it, rank)
        out = torch.empty_like(x)
        assert tbvcoll.all_reduce(x, out), "unsupported"
        outs.append(out)
        ins.append(x)           # keep inputs alive: the caching allocator must not alias them
        if filler is not None:
            filler.sum()
    torch.cuda.synchronize()
    bad, first = 0, None
    for it, out in enumerate(outs):
        acc = gen(it, 0).float()
        for r in range(1, world):
            acc = acc + gen(it, r).float()
        if not torch.equal(out, acc.to(dt)):
            bad += 1
            first = it if first is None else first
    print(f"# rank{rank} dtype={dt} bytes={nb} iters={iters} gap={gap} async={tbvcoll.is_async()} mismatches {bad}/{iters}"
          + (f" first at it={first}" if first is not None else ""), flush=True)
    tbvcoll.hist()
    tbvcoll.fini()
    raise SystemExit(1 if bad else 0)


if __name__ == "__main__":
    main()
