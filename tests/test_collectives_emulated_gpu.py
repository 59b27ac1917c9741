"""The multi-rank collective kernels on ONE GPU: N emulated ranks run as a single
cooperative launch (blockIdx.y = rank), so the push/flag/wait/reduce protocol, the slot
ring and the sequence numbering are exercised for world 2/4/8 without N GPUs.
Oracle: fixed-order fp32 accumulate with one rounding, never another collective library
(same stance as the reference's step4/test_exact.py:3-4)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed, n, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return ((torch.rand(n, generator=g) - 0.5) * 10).to(dtype).to(DEV)


def oracle(ts):
    acc = ts[0].float().clone()
    for t in ts[1:]:
        acc += t.float()
    return acc.to(ts[0].dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ll"])
def test_exact_all_dtypes_sizes(world, algo):
    from libtbvcoll_b200.tbvcoll import Comm
    c = Comm.local(world, 0, cap_bytes=1 << 20)
    c.set_algo(algo)
    try:
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            es = torch.tensor([], dtype=dtype).element_size()
            for nbytes in (16, 57344, 229376, 1048576, 4096 + 16 * 7, 2 * 33):   # incl. odd tails / scalar path
                n = nbytes // es
                ins = [gen(1234 + r, n, dtype) for r in range(world)]
                outs = [torch.empty_like(t) for t in ins]
                assert c.all_reduce_local(ins, outs)
                torch.cuda.synchronize()
                want = oracle(ins)
                for r in range(world):
                    assert torch.equal(outs[r], want), (dtype, nbytes, r)
        assert not c.err()
    finally:
        c.destroy()


@pytest.mark.parametrize("wide,spread,threads", [("1", "0", "0"), ("0", "0", "0"), ("1", "4", "512"), ("1", "2", "64"), ("1", "8", "128")])
def test_ll_packet_width_row_sharing_and_call_trace(monkeypatch, wide, spread, threads):
    """LL packets as one 32-byte store / load per unit (the default) or as two 16-byte ones, a row of the fused
    residual + norm shared by a cluster of 1 / 2 / 4 / 8 CTAs, the plain LL kernel with 64 - 512 threads per CTA:
    all give the bits of the fixed-order oracle followed by the plain norm operator; the per-call trace holds
    ordered device time stamps."""
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.tbvcoll import Comm
    monkeypatch.setenv("TBV_LL_WIDE", wide)
    monkeypatch.setenv("TBV_LL_SPREAD", spread)
    monkeypatch.setenv("TBV_LL_THREADS", threads)
    world = 8
    c = Comm.local(world, 0, cap_bytes=1 << 18)
    c.set_algo("ll")
    try:
        calls = 0
        for T, H in ((5, 4096), (3, 8192), (2, 1024)):
            ins = [gen(900 + r, T * H, torch.bfloat16) for r in range(world)]
            outs = [torch.empty_like(t) for t in ins]
            for _ in range(3):
                assert c.all_reduce_local(ins, outs)
            torch.cuda.synchronize()
            want = oracle(ins)
            assert all(torch.equal(o, want) for o in outs)
            res = gen(77, T * H, torch.bfloat16).view(T, H)
            gamma = gen(78, H, torch.bfloat16)
            xs = [t.view(T, H) for t in ins]
            r_out = [torch.empty(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            ys = [torch.empty(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            for _ in range(2):
                assert c.all_reduce_rmsnorm_local(xs, [res] * world, gamma, 1e-5, r_out, ys)
            torch.cuda.synchronize()
            h = (want.view(T, H).float() + res.float()).to(torch.bfloat16)
            y_want = torch.empty_like(h)
            ops.rmsnorm(h, gamma, 1e-5, out=y_want)
            for r in range(world):
                assert torch.equal(r_out[r], h) and torch.equal(ys[r], y_want), (T, H, r)
            calls += 5
        rows = c.trace(0)
        assert len(rows) == calls and [r[0] for r in rows] == list(range(1, calls + 1))
        for seq, t_enter, t_pushed, t_ready, t_done in rows:
            assert 0 < t_enter <= t_pushed <= t_ready <= t_done, rows
        assert len(c.trace(3, max_rows=2)) == 2 and not c.err()
    finally:
        c.destroy()


@pytest.mark.parametrize("world,algo", [(2, "oneshot"), (8, "oneshot"), (4, "twoshot"), (2, "ll"), (8, "ll")])
def test_stress_back_to_back_no_sync_4_slots(world, algo):
    """Counterpart of step4/test_stress.py:23-42: many calls with no synchronisation in
    between (slot reuse), every output checked afterwards."""
    from libtbvcoll_b200.tbvcoll import Comm
    c = Comm.local(world, 0, cap_bytes=57344)
    c.set_algo(algo)
    iters, n = 300, 57344 // 2
    try:
        ins = [[gen(it * world + r, n, torch.bfloat16) for r in range(world)] for it in range(iters)]
        outs = [[torch.empty_like(t) for t in row] for row in ins]
        for it in range(iters):
            assert c.all_reduce_local(ins[it], outs[it])
        torch.cuda.synchronize()
        bad = sum(0 if all(torch.equal(o, oracle(ins[it])) for o in outs[it]) else 1 for it in range(iters))
        assert bad == 0
        pre, xfer, post, enq, drain, n_calls = c.stats5()
        assert n_calls == iters and xfer >= 0
        c.rails()                                            # per-peer arrival waits: read from the device and reset
        c.hist()
    finally:
        c.destroy()


def test_in_place_unaligned_and_graph_replay():
    from libtbvcoll_b200.tbvcoll import Comm
    world = 4
    c = Comm.local(world, 0, cap_bytes=1 << 16)
    try:
        base = [gen(50 + r, 1001, torch.bfloat16) for r in range(world)]
        views = [b[1:].clone()[0:999] for b in base]            # aligned clones
        un = [torch.empty(1001, dtype=torch.bfloat16, device=DEV)[1:1000] for _ in range(world)]  # 2-byte aligned views
        for u, v in zip(un, views):
            u.copy_(v)
        want = oracle(views)
        assert c.all_reduce_local(un)                            # in place, scalar path
        torch.cuda.synchronize()
        assert all(torch.equal(u, want) for u in un)
        # CUDA graph: sequence numbers live on the device, so a captured call replays correctly
        xs = [gen(70 + r, 4096, torch.bfloat16) for r in range(world)]
        ys = [torch.empty_like(x) for x in xs]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            c.all_reduce_local(xs, ys)                           # warm-up outside capture
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                c.all_reduce_local(xs, ys)
            for rep in range(6):                                 # more replays than slots
                for r in range(world):
                    xs[r].copy_(gen(100 * rep + r, 4096, torch.bfloat16))
                g.replay()
                s.synchronize()
                assert all(torch.equal(y, oracle(xs)) for y in ys)
        assert not c.err()
    finally:
        c.destroy()


@pytest.mark.parametrize("world,T,H", [(2, 8, 4096), (8, 3, 4096), (4, 16, 8192), (2, 1, 1024)])
def test_fused_allreduce_residual_rmsnorm(world, T, H):
    from libtbvcoll_b200.tbvcoll import Comm
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.ops import reference as ref
    c = Comm.local(world, 0, cap_bytes=T * H * 2)
    try:
        xs = [gen(r, T * H, torch.bfloat16).view(T, H) * 0.1 for r in range(world)]
        res = [gen(99, T * H, torch.bfloat16).view(T, H) for _ in range(world)]
        gamma = gen(7, H, torch.bfloat16)
        res_out = [torch.empty_like(x) for x in xs]
        ys = [torch.empty_like(x) for x in xs]
        assert c.all_reduce_rmsnorm_local(xs, res, gamma, 1e-5, res_out, ys)
        torch.cuda.synchronize()
        want_y, want_h = ref.ar_residual_rmsnorm(xs, res[0], gamma, 1e-5)
        # the unfused pipeline (all-reduce, then the add+norm op) must give the same BITS
        summed = [torch.empty_like(x) for x in xs]
        c.all_reduce_local(xs, summed)
        y_unf, h_unf = ops.add_rmsnorm(summed[0].clone(), res[0].clone(), gamma, 1e-5)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(res_out[r], want_h)
            assert torch.equal(ys[r], y_unf)
            assert (ys[r].float() - want_y.float()).abs().max().item() <= 2 ** -6 * want_y.float().abs().max().item()
    finally:
        c.destroy()


@pytest.mark.parametrize("world,T,H,K", [(2, 8, 512, 256), (4, 5, 1024, 1024), (2, 32, 4096, 2048), (2, 130, 512, 512),
                                         (8, 8, 4096, 512), (4, 8, 8192, 1024), (8, 1, 4096, 1792)])
def test_fused_gemm_allreduce_residual_rmsnorm_emulated(world, T, H, K):
    """Row-parallel GEMM whose epilogue stores LL packets into every rank's memory while finisher CTAs
    reduce + residual + RMSNorm the rows as they land, all in one kernel; ranks emulated on one GPU.
    Must equal the unfused pipeline (GEMM, all-reduce, add+norm op) bit for bit."""
    from libtbvcoll_b200.tbvcoll import Comm
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.ops import reference as ref
    c = Comm.local(world, 0, cap_bytes=T * H * 2)
    try:
        g = torch.Generator().manual_seed(5)
        xs = [(torch.randn(T, K, generator=g)).to(torch.bfloat16).to(DEV) for _ in range(world)]
        ws = [(torch.randn(H, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV) for _ in range(world)]
        res0 = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
        gamma = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(DEV)
        # unfused pipeline on the same kernels: GEMM per rank, exact all-reduce, add + norm
        parts = [ops.gemm(x, w) for x, w in zip(xs, ws)]
        summed = [torch.empty_like(p) for p in parts]
        assert c.all_reduce_local(parts, summed)
        y_unf, h_unf = ops.add_rmsnorm(summed[0].clone(), res0.clone(), gamma, 1e-5)
        torch.cuda.synchronize()
        for rep in range(6):      # more calls than slots: slot ring and sequence numbers advance
            res = [res0.clone() for _ in range(world)]
            ys = [torch.zeros(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            ok = c.gemm_all_reduce_rmsnorm_local(xs, ws, res, gamma, 1e-5, ys)
            assert ok, "the fused kernel declined a shape it should take"
            torch.cuda.synchronize()
            assert not c.err()
            for r in range(world):
                assert torch.equal(res[r], h_unf), (rep, r)
                assert torch.equal(ys[r], y_unf), (rep, r)
        partials = [ref.gemm(x, w).to(torch.bfloat16) for x, w in zip(xs, ws)]
        want_y, want_h = ref.ar_residual_rmsnorm(partials, res0, gamma, 1e-5)
        tol_h = 2 ** -6 * want_h.float().abs().max().item()
        assert (h_unf.float() - want_h.float()).abs().max().item() <= tol_h
        assert (y_unf.float() - want_y.float()).abs().max().item() <= 2 ** -5 * want_y.float().abs().max().item()
    finally:
        c.destroy()


def test_fused_gemm_allreduce_declines_large_messages_on_shape_alone(monkeypatch):
    """Above the LL packet limit the call is declined (the caller composes GEMM + collective); the answer
    depends on the shape and the knobs only, so all ranks agree on it."""
    from libtbvcoll_b200.tbvcoll import Comm
    monkeypatch.setenv("TBV_LL_MAX", str(256 << 10))
    T, H, K, world = 128, 4096, 256, 2
    c = Comm.local(world, 0, cap_bytes=T * H * 2)
    try:
        xs = [torch.zeros(T, K, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        ws = [torch.zeros(H, K, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        res = [torch.zeros(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        ys = [torch.zeros(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        gamma = torch.ones(H, dtype=torch.bfloat16, device=DEV)
        assert c.gemm_all_reduce_rmsnorm_local(xs, ws, res, gamma, 1e-5, ys) is False
        assert not c.err()
    finally:
        c.destroy()


@pytest.mark.parametrize("kind", ["oneshot", "ll", "twoshot", "fused_norm", "fused_norm_ll", "fused_gemm"])
def test_device_watchdog_when_one_emulated_rank_never_calls(kind):
    """Failure detection on ONE GPU, made on the host: one emulated rank sits out a call (its CTAs
    return before pushing anything).  The others' bounded waits run out after the watchdog period, the
    kernel ENDS, the error is sticky, names the silent rank, later calls are refused, and the CUDA
    context stays usable.  Nothing faults or traps."""
    import time
    from libtbvcoll_b200.tbvcoll import Comm
    world, silent = 4, 2
    T, H, K = 4, 1024, 256
    c = Comm.local(world, 0, cap_bytes=1 << 20)
    try:
        c.set_wdog(0.05)
        xs = [gen(r, T * H, torch.bfloat16).view(T, H) for r in range(world)]
        outs = [torch.empty_like(x) for x in xs]
        res = [gen(9, T * H, torch.bfloat16).view(T, H) for _ in range(world)]
        gamma = gen(7, H, torch.bfloat16)
        if kind in ("oneshot", "ll", "twoshot"):
            c.set_algo(kind)
        elif kind == "fused_norm":
            c.set_algo("oneshot")
        assert c.all_reduce_local(xs, outs) if kind in ("oneshot", "ll", "twoshot") else True    # a good call first
        torch.cuda.synchronize()
        assert not c.err()
        c.mute_rank(silent, 1)
        t0 = time.perf_counter()
        if kind in ("oneshot", "ll", "twoshot"):
            assert c.all_reduce_local(xs, outs)
        elif kind in ("fused_norm", "fused_norm_ll"):
            assert c.all_reduce_rmsnorm_local(xs, res, gamma, 1e-5, [torch.empty_like(x) for x in xs], outs)
        else:
            a = [gen(20 + r, T * K, torch.bfloat16).view(T, K) for r in range(world)]
            w = [gen(30 + r, H * K, torch.bfloat16).view(H, K) * 0.05 for r in range(world)]
            assert c.gemm_all_reduce_rmsnorm_local(a, w, res, gamma, 1e-5, outs)
        torch.cuda.synchronize()                        # returns: every wait is bounded
        elapsed = time.perf_counter() - t0
        assert 0.04 < elapsed < 5.0, elapsed
        assert c.err()                                   # sticky
        last = c.last_error()
        assert last["code"] == 1 and last["peer"] == silent, last
        with pytest.raises(RuntimeError):
            c.all_reduce_local(xs, outs)                 # refused: "previous collective failed: unrecoverable"
        assert float((torch.ones(4, device=DEV) * 4).sum()) == 16.0     # the context is alive
    finally:
        c.destroy()


def test_stream_wait_value_mode_and_its_host_watchdog(monkeypatch):
    """TBV_STREAMWAIT=1, the host-driven debug mode: push half, one stream wait-value operation per (source, channel)
    on the receiver's own flag words, reduce half.  Same bits as the fixed-order oracle, also in place and after graph
    replays have advanced the device's sequence number.  Then one emulated rank never publishes: the stream blocks,
    the HOST's bound runs out, the missing source is named, the host stores the awaited value so that the stream
    drains, the communicator is failed and the context stays usable.  Nothing faults or spins without a limit."""
    import time
    from libtbvcoll_b200.tbvcoll import Comm
    monkeypatch.setenv("TBV_STREAMWAIT", "1")
    world, silent = 4, 1
    c = Comm.local(world, 0, cap_bytes=1 << 20)
    try:
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            es = torch.tensor([], dtype=dtype).element_size()
            for nbytes in (16, 57344, 1 << 20, 4096 + 16 * 7, 2 * 33):
                ins = [gen(500 + r, nbytes // es, dtype) for r in range(world)]
                outs = [torch.empty_like(t) for t in ins]
                assert c.all_reduce_local(ins, outs)
                torch.cuda.synchronize()
                want = oracle(ins)
                assert all(torch.equal(o, want) for o in outs), (dtype, nbytes)
        ins = [gen(600 + r, 4096, torch.bfloat16) for r in range(world)]
        want = oracle(ins)
        assert c.all_reduce_local(ins, ins)                  # in place
        torch.cuda.synchronize()
        assert all(torch.equal(t, want) for t in ins) and not c.err()
        rows = c.trace(0)
        assert rows and all(0 < r[1] <= r[2] <= r[3] <= r[4] for r in rows)
        c.set_wdog(0.2)
        c.mute_rank(silent, 1)
        xs = [gen(700 + r, 8192, torch.bfloat16) for r in range(world)]
        outs = [torch.empty_like(t) for t in xs]
        t0 = time.perf_counter()
        with pytest.raises(RuntimeError):
            c.all_reduce_local(xs, outs)
        elapsed = time.perf_counter() - t0
        assert 0.15 < elapsed < 5.0, elapsed
        torch.cuda.synchronize()                             # the stream has drained
        assert c.err()
        last = c.last_error()
        assert last["code"] == 1 and last["peer"] == silent and last["where"] == 4, last
        with pytest.raises(RuntimeError):
            c.all_reduce_local(xs, outs)
        assert float((torch.ones(4, device=DEV) * 4).sum()) == 16.0
    finally:
        c.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_sequence_stamp_diagnostic(world, monkeypatch):
    """TBV_TAG=1: every flag is preceded by a sequence stamp in a word of its own; the receiver compares
    it after the flag.  A message that fills the slot to the last byte is still exact (the stamp does
    not live inside the payload), every flag wait is checked, none mismatches."""
    from libtbvcoll_b200.tbvcoll import Comm
    monkeypatch.setenv("TBV_TAG", "1")
    nbytes = 57344
    c = Comm.local(world, 0, cap_bytes=nbytes)          # capacity == message size
    try:
        n = nbytes // 2
        calls = 0
        for algo in ("oneshot", "twoshot"):
            c.set_algo(algo)
            for it in range(5):
                ins = [gen(1000 * it + r, n, torch.bfloat16) for r in range(world)]
                outs = [torch.empty_like(t) for t in ins]
                assert c.all_reduce_local(ins, outs)
                torch.cuda.synchronize()
                assert all(torch.equal(o, oracle(ins)) for o in outs), (algo, it)
                calls += 1
        T, H = 7, 4096
        c.set_algo("oneshot")
        xs = [gen(r, T * H, torch.bfloat16).view(T, H) * 0.1 for r in range(world)]
        res = [gen(99, T * H, torch.bfloat16).view(T, H) for _ in range(world)]
        assert c.all_reduce_rmsnorm_local(xs, res, gen(7, H, torch.bfloat16), 1e-5, [torch.empty_like(x) for x in xs],
                                          [torch.empty_like(x) for x in xs])
        torch.cuda.synchronize()
        checked, bad = c.tag_counts()
        assert bad == 0 and checked >= calls * world * (world - 1)
        c.hist()                                             # prints tag_checked / tag_bad
        assert not c.err()
    finally:
        c.destroy()
    monkeypatch.delenv("TBV_TAG")
    c = Comm.local(world, 0, cap_bytes=nbytes)
    try:
        ins = [gen(r, nbytes // 2, torch.bfloat16) for r in range(world)]
        assert c.all_reduce_local(ins)
        torch.cuda.synchronize()
        assert c.tag_counts() == (0, 0)                      # off by default: nothing stamped, nothing compared
    finally:
        c.destroy()


def test_mixed_alignment_takes_the_same_kernel():
    """A tensor that is not 16-byte aligned is accessed element by element inside the SAME kernel and
    channel partition (the choice depends on the byte count only), so ranks whose tensors sit at
    different alignments still run one protocol."""
    from libtbvcoll_b200.tbvcoll import Comm
    world, n = 4, 4096                                     # 8192 bytes: a multiple of 16
    c = Comm.local(world, 0, cap_bytes=1 << 16)
    try:
        for algo in ("ll", "oneshot", "twoshot"):
            c.set_algo(algo)
            base = [torch.empty(n + 8, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            ins = [b[(1 if r % 2 else 0):][:n] for r, b in enumerate(base)]      # odd ranks: 2-byte aligned views
            for r, t in enumerate(ins):
                t.copy_(gen(40 + r, n, torch.bfloat16))
            outs = [torch.empty(n + 8, dtype=torch.bfloat16, device=DEV)[(0 if r % 2 else 3):][:n] for r in range(world)]
            assert c.all_reduce_local(ins, outs)
            torch.cuda.synchronize()
            want = oracle([t.clone() for t in ins])
            assert all(torch.equal(o, want) for o in outs), algo
        assert not c.err()
    finally:
        c.destroy()


@pytest.mark.parametrize("world,T,H,K", [(2, 64, 512, 256), (4, 128, 1024, 512), (2, 512, 4096, 1024), (8, 256, 256, 128)])
def test_gemm_reduce_scatter_emulated(world, T, H, K):
    """GEMM whose tile epilogues scatter into the owners' slot memory, then reduce (+ residual + norm)."""
    from libtbvcoll_b200.tbvcoll import Comm
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.ops import reference as ref
    rpr = T // world
    c = Comm.local(world, 0, cap_bytes=rpr * H * 2)
    try:
        g = torch.Generator().manual_seed(6)
        xs = [torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV) for _ in range(world)]
        ws = [(torch.randn(H, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV) for _ in range(world)]
        gamma = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(DEV)
        res0 = [torch.randn(rpr, H, generator=g).to(torch.bfloat16).to(DEV) for _ in range(world)]
        partials = [ops.gemm(x, w, splits=1) for x, w in zip(xs, ws)]          # same kernel arithmetic, no collective
        torch.cuda.synchronize()
        total = oracle(partials)
        for rep in range(3):
            outs = [torch.zeros(rpr, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            assert c.gemm_reduce_scatter_local(xs, ws, outs=outs)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(outs[r], total[r * rpr:(r + 1) * rpr]), (rep, r)
            res = [t.clone() for t in res0]
            ys = [torch.zeros(rpr, H, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            assert c.gemm_reduce_scatter_local(xs, ws, residuals=res, gamma=gamma, eps=1e-5, ys=ys)
            torch.cuda.synchronize()
            for r in range(world):
                y2, h2 = ops.add_rmsnorm(total[r * rpr:(r + 1) * rpr].clone(), res0[r].clone(), gamma, 1e-5)
                assert torch.equal(res[r], h2) and torch.equal(ys[r], y2)       # bit-identical to the unfused pipeline
        assert not c.err()
        want = ref.gemm(xs[0], ws[0])
        assert (partials[0].float() - want).abs().max().item() <= 0.01 * want.abs().max().item() + 1e-3
    finally:
        c.destroy()


@pytest.mark.parametrize("world,rows,M,K", [(2, 32, 256, 128), (4, 64, 384, 512), (2, 256, 1024, 2048), (8, 16, 128, 64)])
def test_allgather_gemm_emulated(world, rows, M, K):
    from libtbvcoll_b200.tbvcoll import Comm
    from libtbvcoll_b200 import ops
    c = Comm.local(world, 0, cap_bytes=rows * K * 2)
    try:
        g = torch.Generator().manual_seed(8)
        xs = [torch.randn(rows, K, generator=g).to(torch.bfloat16).to(DEV) for _ in range(world)]
        ws = [(torch.randn(M, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV) for _ in range(world)]
        full = torch.cat(xs, 0)
        for rep in range(3):
            ys = [torch.zeros(world * rows, M, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            assert c.allgather_gemm_local(xs, ws, ys)
            torch.cuda.synchronize()
            for r in range(world):
                want = ops.gemm(full, ws[r], splits=1)
                torch.cuda.synchronize()
                assert torch.equal(ys[r], want), (rep, r)
        assert not c.err()
    finally:
        c.destroy()


def test_allgather_gemm_after_destroy_and_create_with_the_same_shapes():
    """The gathered-chunk tensor maps belong to their communicator: a second communicator created after
    the first was destroyed (very likely at the same heap address, with the same shapes) builds its own
    maps over its own slot memory."""
    from libtbvcoll_b200.tbvcoll import Comm
    from libtbvcoll_b200 import ops
    world, rows, M, K = 2, 32, 256, 128
    g = torch.Generator().manual_seed(8)
    xs = [torch.randn(rows, K, generator=g).to(torch.bfloat16).to(DEV) for _ in range(world)]
    ws = [(torch.randn(M, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV) for _ in range(world)]
    full = torch.cat(xs, 0)
    want = [ops.gemm(full, w, splits=1) for w in ws]
    for life in range(3):
        c = Comm.local(world, 0, cap_bytes=rows * K * 2)
        junk = torch.empty(1 << 20, dtype=torch.uint8, device=DEV) if life % 2 else None   # shift the allocator between lives
        try:
            ys = [torch.zeros(world * rows, M, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
            assert c.allgather_gemm_local(xs, ws, ys)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(ys[r], want[r]), (life, r)
            assert not c.err()
        finally:
            c.destroy()
        del junk
