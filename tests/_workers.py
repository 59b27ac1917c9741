"""Child-process bodies for multi-rank tests (spawned; must be importable)."""
import os
import sys
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_ranks(fn, world, *args, timeout=120, env=None):
    """Run fn(rank, world, *args) in `world` spawned processes; returns the list of results.
    A worker that raises makes the test fail with its traceback; a worker that hangs is
    killed after `timeout` (by exact pid)."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = []
    old = {}
    if env:
        for k, v in env.items():
            old[k] = os.environ.get(k)
            os.environ[k] = str(v)
    try:
        for r in range(world):
            p = ctx.Process(target=_entry, args=(fn, r, world, q, args))
            p.start()
            procs.append(p)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    results = {}
    try:
        for _ in range(world):
            r, ok, val = q.get(timeout=timeout)
            if not ok:
                raise AssertionError(f"rank {r} failed:\n{val}")
            results[r] = val
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]


def _entry(fn, rank, world, q, args):
    try:
        import torch
        torch.set_num_threads(1)
        q.put((rank, True, fn(rank, world, *args)))
    except BaseException:
        q.put((rank, False, traceback.format_exc()))


# ---- CPU backend ---------------------------------------------------------------------
def oracle_sum(tensors):
    """fixed-order (rank 0..N-1) fp32 accumulate, one rounding"""
    import torch
    acc = tensors[0].float().clone()
    for t in tensors[1:]:
        acc += t.float()
    return acc.to(tensors[0].dtype)


def gen(seed, shape, dtype, device="cpu"):
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype).to(device)


def cpu_async_stream(rank, world, port, iters, nslot, dtype_name, shape):
    import torch
    os.environ["TBV_NSLOT"] = str(nslot)
    from libtbvcoll_b200 import tbvcoll
    dtype = getattr(torch, dtype_name)
    tbvcoll.init_n(rank, world, -1, "127.0.0.1", port, cap_bytes=1 << 20)
    assert tbvcoll.is_async()
    ins, outs = [], []
    for it in range(iters):
        x = gen(it * world + rank, shape, dtype)
        out = torch.empty_like(x)
        assert tbvcoll.all_reduce(x, out)
        ins.append(x)
        outs.append(out)
    tbvcoll.synchronize()
    bad = 0
    for it, out in enumerate(outs):
        ref = oracle_sum([gen(it * world + r, shape, dtype) for r in range(world)])
        if not torch.equal(out, ref):
            bad += 1
    pre, xfer, post, enq, drain, n = tbvcoll.stats5()
    import hashlib
    h = hashlib.sha256(b"".join(o.view(torch.int16 if o.element_size() == 2 else torch.int32).numpy().tobytes() for o in outs)).hexdigest()
    tbvcoll.fini()
    return {"bad": bad, "n": n, "hash": h}


def cpu_contract(rank, world, port):
    import torch
    from libtbvcoll_b200 import tbvcoll
    tbvcoll.init_n(rank, world, -1, "127.0.0.1", port, cap_bytes=8192)
    tbvcoll.init_n(rank, world, -1, "127.0.0.1", port, cap_bytes=8192)  # idempotent
    res = {}
    res["cap"] = tbvcoll.cap()
    res["zero"] = tbvcoll.all_reduce(torch.empty(0))
    res["big"] = tbvcoll.all_reduce(torch.zeros(8192))            # 32 KiB > cap -> False
    res["int"] = tbvcoll.all_reduce(torch.zeros(4, dtype=torch.int32))
    res["noncontig"] = tbvcoll.all_reduce(torch.zeros(4, 4).t())
    res["badout"] = tbvcoll.all_reduce(torch.zeros(4), torch.zeros(5))
    t = torch.full((7,), float(rank + 1))
    res["inplace"] = tbvcoll.all_reduce(t)
    tbvcoll.synchronize()
    res["val"] = t.tolist()
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        x = gen(100 + rank, (33,), dt)
        o = torch.empty_like(x)
        assert tbvcoll.all_reduce(x, o)
        tbvcoll.synchronize()
        ref = oracle_sum([gen(100 + r, (33,), dt) for r in range(world)])
        res[str(dt)] = bool(torch.equal(o, ref))
    # raw_fn: the C function itself
    fn = tbvcoll.raw_fn()
    import ctypes
    y = torch.full((16,), 2.0)
    rc = fn(ctypes.c_void_p(y.data_ptr()), None, 64, 0, None)
    tbvcoll.synchronize()
    res["raw"] = (rc, y[0].item())
    rc = fn(ctypes.c_void_p(y.data_ptr()), None, 1 << 20, 0, None)
    res["raw_big"] = rc
    res["err"] = tbvcoll.err()
    tbvcoll.fini()
    return res


def cpu_rs_ag(rank, world, port):
    import torch
    from libtbvcoll_b200 import tbvcoll
    c = tbvcoll.Comm(rank, world, -1, "127.0.0.1", port, cap_bytes=1 << 16)
    n = 96
    full = [gen(7 + r, (world * n,), torch.bfloat16) for r in range(world)]
    out = torch.empty(n, dtype=torch.bfloat16)
    assert c.reduce_scatter(full[rank], out)
    c.synchronize()
    ref = oracle_sum(full)[rank * n:(rank + 1) * n]
    ok_rs = bool(torch.equal(out, ref))
    g = torch.empty(world * n, dtype=torch.bfloat16)
    assert c.all_gather(out, g)
    c.synchronize()
    ok_ag = bool(torch.equal(g, oracle_sum(full)))
    c.destroy()
    return ok_rs, ok_ag


def cpu_peer_skips(rank, world, port):
    """rank 1 drops one call on the host: rank 0's bounded wait must expire, the call must
    complete with an error and later calls must be refused."""
    import time
    import torch
    os.environ["TBV_WDOG"] = "0.3"
    from libtbvcoll_b200 import tbvcoll
    c = tbvcoll.Comm(rank, world, -1, "127.0.0.1", port, cap_bytes=4096)
    t = torch.ones(16)
    assert c.all_reduce(t)
    c.synchronize()
    res = {"first": t[0].item()}
    if rank == 1:
        c.skip_next(1)
    t0 = time.time()
    c.all_reduce(torch.ones(16))
    failed = False
    try:
        c.synchronize()
    except RuntimeError:
        failed = True
    res["elapsed"] = time.time() - t0
    res["failed"] = failed
    res["err"] = c.err()
    res["last"] = c.last_error()
    if rank == 0:
        try:
            c.all_reduce(torch.ones(16))
            res["refused"] = False
        except RuntimeError:
            res["refused"] = True
    time.sleep(0.5)
    c.destroy()
    return res


def cpu_never_joins(rank, world, port):
    """world=2 but rank 1 never starts: init must fail after TBV_INIT_TIMEOUT, not hang."""
    import time
    os.environ["TBV_INIT_TIMEOUT"] = "1.0"
    from libtbvcoll_b200 import tbvcoll
    t0 = time.time()
    try:
        tbvcoll.Comm(0, 2, -1, "127.0.0.1", port, cap_bytes=4096)
        return {"raised": False}
    except RuntimeError:
        return {"raised": True, "elapsed": time.time() - t0}
