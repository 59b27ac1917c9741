#!/usr/bin/env python3
"""Bit-exactness check on real ranks — the role of the reference's step4/test_exact.py:15-38.

Every rank regenerates ALL ranks' inputs from seeds (1234 + rank), so the expected result is
computed locally with a fixed-order fp32 accumulation and one rounding; no other collective
library is the oracle.  fp32 / bf16 / fp16 x {57344, 229376, 1048576} bytes, out of place.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m libtbvcoll_b200.launch.check_exact
    env: PORT (18997), CAP, TBV_ALGO, TBV_NSLOT, ...
"""
import os

import torch

from libtbvcoll_b200 import tbvcoll


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", "2"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    tbvcoll.init_n(rank, world, local, os.environ.get("PEER_IP", "127.0.0.1"), int(os.environ.get("PORT", "18997")),
                   int(os.environ.get("CAP", str(1 << 20))))
    bad = 0
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        es = torch.tensor([], dtype=dt).element_size()
        for nb in (57344, 229376, 1048576):
            n = nb // es
            gens = [torch.Generator(device="cuda").manual_seed(1234 + r) for r in range(world)]
            fs = [((torch.rand(n, generator=g, device="cuda") - 0.5) * 10).to(dt) for g in gens]
            out = torch.empty_like(fs[rank])
            assert tbvcoll.all_reduce(fs[rank], out), "unsupported"
            torch.cuda.synchronize()
            acc = fs[0].float()
            for f in fs[1:]:
                acc = acc + f.float()
            ref = acc.to(dt)
            same = torch.equal(out, ref)
            bad += 0 if same else 1
            if rank == 0:
                print(f"{str(dt):16s} {nb:8d} B  equal={same}  max|diff|={(out.float() - ref.float()).abs().max().item():.3e}", flush=True)
    tbvcoll.fini()
    raise SystemExit(1 if bad else 0)


if __name__ == "__main__":
    main()
