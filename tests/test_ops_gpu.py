"""Numerics of every sm_100a operator against a plain PyTorch fp32 statement of the same math."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from libtbvcoll_b200 import ops as o
    o.lib()
    return o


from libtbvcoll_b200.ops import reference as ref  # noqa: E402

DEV = "cuda"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("N,M,K,splits", [
    (1, 128, 64, 1), (8, 256, 512, 1), (16, 4096, 2048, 0), (7, 384, 4096, 2), (33, 512, 1024, 4), (64, 4096, 7168, 0),
    (8, 6144, 4096, 0), (200, 256, 320, 1), (300, 640, 1088, 1), (512, 1024, 2048, 1), (5, 16032, 512, 1), (24, 128, 8192, 8),
])
def test_gemm_matches_fp32(ops, N, M, K, splits):
    x, w = rnd(N, K, seed=1), rnd(M, K, scale=0.05, seed=2)
    y = ops.gemm(x, w, splits=splits)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    want = ref.gemm(x, w)
    err = (y.float() - want).abs().max().item()
    tol = 0.01 * want.abs().max().item() + 1e-3
    assert err <= tol, (err, tol, ops.gemm_config(M, N, K, splits))
    # split-K is deterministic: same bits on a second run
    y2 = ops.gemm(x, w, splits=splits)
    assert torch.equal(y, y2)


@pytest.fixture
def streamk_everywhere(ops):
    """The evenly-split decode GEMM for every shape it can take (normally only large weight matrices)."""
    ops.gemm_streamk_min_bytes(0)
    yield
    ops.gemm_streamk_min_bytes(None)


def _elementwise_close(y, want, K):
    """Per-element check: |err| <= bf16 rounding of the result + accumulated input rounding, NOT a fraction of the
    largest output — a wrong K tail on a small-magnitude element must not hide behind a large one."""
    err = (y.float() - want).abs()
    bound = 2.0 ** -7 * want.abs() + 2.0 ** -8 * math.sqrt(K) * 0.05 + 1e-3
    bad = err > bound
    assert not bool(bad.any()), (int(bad.sum()), err.max().item())


@pytest.mark.parametrize("N,M,K,bias", [(8, 4096, 4096, False), (1, 2048, 5120, True), (64, 1024, 9472, False), (13, 4200, 2056, True),
                                        (16, 28672, 1024, False), (33, 640, 16384, True)])
def test_gemm_streamk_matches_fp32(ops, streamk_everywhere, N, M, K, bias):
    """Work split evenly over the SMs: tiles whose K range is shared by several CTAs are summed through global
    scratch in a fixed order.  Ragged feature / K edges, one to 64 tokens, strided output, bias; deterministic;
    correct under CUDA-graph replay (the finishing CTAs clear the flags they consumed)."""
    x, w = rnd(N, K, seed=31), rnd(M, K, scale=0.05, seed=32)
    b = rnd(M, seed=33) if bias else None
    outbuf = torch.zeros(N + 2, M + 64, dtype=torch.bfloat16, device=DEV)
    y = ops.gemm(x, w, out=outbuf[:N, :M], bias=b)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    want = ref.gemm(x, w, b)
    _elementwise_close(y, want, K)
    assert outbuf[:, M:].abs().max().item() == 0 and outbuf[N:].abs().max().item() == 0
    y1 = y.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            ops.gemm(x, w, out=outbuf[:N, :M], bias=b)
            ops.gemm(x, w, out=outbuf[:N, :M], bias=b)
        for _ in range(3):
            outbuf.zero_()
            g.replay()
            s.synchronize()
            assert torch.equal(outbuf[:N, :M], y1)            # same bits on every replay
    torch.cuda.current_stream().wait_stream(s)
    y_tile = ops.gemm(x, w, bias=b, splits=1)                   # the tile kernel on the same problem
    torch.cuda.synchronize()
    assert (y_tile.float() - y1.float()).abs().max().item() <= 0.01 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("N,I,K", [(8, 14336, 4096), (2, 1280, 8192), (64, 2048, 4160)])
def test_gemm_streamk_silu_mul(ops, streamk_everywhere, N, I, K):
    x, wg, wu = rnd(N, K, seed=34), rnd(I, K, scale=0.05, seed=35), rnd(I, K, scale=0.05, seed=36)
    fused = ops.gemm(x, ops.interleave_gate_up(wg, wu), epi=ops.EPI_SILU_MUL)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    want = ref.silu_mul(torch.cat((ref.gemm(x, wg), ref.gemm(x, wu)), -1))
    assert (fused.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-3
    assert torch.equal(fused, ops.gemm(x, ops.interleave_gate_up(wg, wu), epi=ops.EPI_SILU_MUL))


def test_gemm_ragged_k_per_element(ops):
    """The tile kernel on a K that is not a multiple of the 64-wide block, checked element by element."""
    N, M, K = 9, 384, 1096
    x, w = rnd(N, K, seed=41), rnd(M, K, scale=0.05, seed=42)
    w[:, -8:] *= 40.0                                            # the K tail carries real weight: dropping it must show
    for splits in (1, 2, 4):
        y = ops.gemm(x, w, splits=splits)
        torch.cuda.synchronize()
        _elementwise_close(y, ref.gemm(x, w), K)


def test_gemm_bias_and_strided_rows(ops):
    N, M, K = 12, 256, 512
    big = rnd(N, K + 64, seed=3)
    x = big[:, :K]                       # row stride K + 64
    w, b = rnd(M, K, scale=0.05, seed=4), rnd(M, seed=5)
    outbuf = torch.zeros(N, M + 128, dtype=torch.bfloat16, device=DEV)
    y = ops.gemm(x, w, out=outbuf[:, :M], bias=b)
    torch.cuda.synchronize()
    want = ref.gemm(x, w, b)
    assert (y.float() - want).abs().max().item() <= 0.01 * want.abs().max().item() + 1e-3
    assert outbuf[:, M:].abs().max().item() == 0


@pytest.mark.parametrize("N,I,K,splits", [(8, 1024, 512, 1), (3, 7168, 4096, 0), (40, 256, 2048, 2), (260, 512, 256, 1)])
def test_gemm_silu_mul_epilogue_equals_unfused_bits(ops, N, I, K, splits):
    x, wg, wu = rnd(N, K, seed=6), rnd(I, K, scale=0.05, seed=7), rnd(I, K, scale=0.05, seed=8)
    fused = ops.gemm(x, ops.interleave_gate_up(wg, wu), epi=ops.EPI_SILU_MUL, splits=splits)
    gu = ops.gemm(x, torch.cat((wg, wu), 0).contiguous(), splits=splits)
    unfused = ops.silu_mul(gu)
    torch.cuda.synchronize()
    assert torch.equal(fused, unfused)
    want = ref.silu_mul(torch.cat((ref.gemm(x, wg), ref.gemm(x, wu)), -1))
    assert (fused.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("mode", ["2", "3"])                    # 128-token tiles (two accumulators) / 256-token tiles
@pytest.mark.parametrize("N,M,K,bias", [(384, 256, 64, False), (512, 1024, 2048, True), (1000, 656, 1088, True), (4096, 1536, 512, False),
                                        (777, 16, 192, False), (2500, 4096, 4096, False)])
def test_gemm_many_tokens_persistent_kernel(ops, persist_mode, N, M, K, bias, mode):
    """384 tokens and more (and no split hint) can take the persistent kernel: tokens on the UMMA M axis,
    TMEM fully used.  Ragged token / feature / K edges, a strided output and the bias are covered."""
    persist_mode(int(mode))                                     # forced: also where the tile count fills the SMs badly
    x, w = rnd(N, K, seed=21), rnd(M, K, scale=0.05, seed=22)
    b = rnd(M, seed=23) if bias else None
    outbuf = torch.zeros(N + 3, M + 64, dtype=torch.bfloat16, device=DEV)
    y = ops.gemm(x, w, out=outbuf[:N, :M], bias=b)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    want = ref.gemm(x, w, b)
    err = (y.float() - want).abs().max().item()
    assert err <= 0.01 * want.abs().max().item() + 1e-3, err
    assert outbuf[:, M:].abs().max().item() == 0 and outbuf[N:].abs().max().item() == 0
    y2 = ops.gemm(x, w, bias=b)
    assert torch.equal(y2, y)                                   # deterministic
    y_dec = ops.gemm(x, w, bias=b, splits=1)                    # the decode-form kernel on the same problem
    assert (y_dec.float() - y.float()).abs().max().item() <= 0.01 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("mode", ["2", "3"])
@pytest.mark.parametrize("N,I,K", [(384, 128, 256), (1030, 1288, 1024), (4096, 512, 4096)])
def test_gemm_many_tokens_silu_mul(ops, persist_mode, N, I, K, mode):
    persist_mode(int(mode))
    x, wg, wu = rnd(N, K, seed=24), rnd(I, K, scale=0.05, seed=25), rnd(I, K, scale=0.05, seed=26)
    fused = ops.gemm(x, ops.interleave_gate_up(wg, wu), epi=ops.EPI_SILU_MUL)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    want = ref.silu_mul(torch.cat((ref.gemm(x, wg), ref.gemm(x, wu)), -1))
    assert (fused.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-3
    unfused = ops.silu_mul(ops.gemm(x, torch.cat((wg, wu), 0).contiguous()))
    assert (fused.float() - unfused.float()).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-3


@pytest.mark.parametrize("T,H", [(1, 4096), (9, 4096), (5, 8192), (3, 1024), (2, 12288), (4, 264)])
def test_rmsnorm_and_add_rmsnorm_bit_exact(ops, T, H):
    x, r, g = rnd(T, H, seed=9), rnd(T, H, seed=10), rnd(H, seed=11)
    y = ops.rmsnorm(x, g, 1e-5)
    want = ref.rmsnorm(x, g, 1e-5)
    assert (y.float() - want.float()).abs().max().item() <= 2 ** -6 * want.float().abs().max().item()
    y2, h2 = ops.add_rmsnorm(x.clone(), r.clone(), g, 1e-5)
    want2, hw = ref.add_rmsnorm(x, r, g, 1e-5)
    assert torch.equal(h2, hw)
    assert (y2.float() - want2.float()).abs().max().item() <= 2 ** -6 * want2.float().abs().max().item()


def test_rope_kv_writes_cache_and_matches_hf_rotation(ops):
    T, nq, nkv, D, bs, nblocks = 11, 8, 2, 128, 16, 6
    qkv = rnd(T, (nq + 2 * nkv) * D, seed=12)
    pos = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    cs = ops.rope_cos_sin(D, 64, 5e5, DEV)
    slots = torch.randperm(bs * nblocks)[:T].to(DEV)
    slots[2] = -1
    kc = torch.zeros(bs * nblocks, nkv, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    orig = qkv.clone().view(T, nq + 2 * nkv, D)
    ops.rope_kv(qkv, pos, cs, slots, kc, vc, nq, nkv, D)
    got = qkv.view(T, nq + 2 * nkv, D)
    want = ref.rope(orig[:, : nq + nkv], pos, cs)
    assert torch.equal(got[:, : nq + nkv], want)
    assert torch.equal(got[:, nq + nkv:], orig[:, nq + nkv:])
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        assert torch.equal(kc[s], got[t, nq: nq + nkv]) and torch.equal(vc[s], orig[t, nq + nkv:])
    assert kc.abs().sum(dim=(1, 2)).ne(0).sum().item() == T - 1


def test_silu_mul_embedding_argmax(ops):
    x = rnd(5, 2 * 1000, seed=13)
    assert torch.equal(ops.silu_mul(x), ref.silu_mul(x))
    table = rnd(300, 256, seed=14)
    ids = torch.tensor([0, 299, 100, 1000, 450, 399], device=DEV)
    e = ops.embedding(ids, table, vocab_start=100)
    want = torch.zeros(6, 256, dtype=torch.bfloat16, device=DEV)
    want[1], want[2], want[5] = table[199], table[0], table[299]
    assert torch.equal(e, want)
    logits = rnd(7, 128256, seed=15)
    logits[3, 77] = logits[3, 90000] = 50.0      # a tie: the lower index must win
    ws = ops.argmax_workspace(7, DEV)
    for _ in range(2):                            # second launch checks that the tickets were reset
        v, i = ops.argmax(logits, ws, index_offset=1000)
        wv, wi = ref.argmax_first(logits)
        assert torch.equal(i, wi + 1000) and torch.equal(v, wv)
    T, world = 2, 3
    idx_off, rec = ops.cand_layout(T)
    packed = torch.zeros(world, rec, dtype=torch.uint8, device=DEV)
    vals = [[1.0, 5.0], [3.0, 5.0], [2.0, 1.0]]
    idx = [[10, 70], [20, 30], [5, 6]]
    for r in range(world):
        packed[r, : T * 4] = torch.tensor(vals[r], dtype=torch.float32).view(torch.uint8).to(DEV)
        packed[r, idx_off: idx_off + T * 8] = torch.tensor(idx[r], dtype=torch.int64).view(torch.uint8).to(DEV)
    out = torch.empty(T, dtype=torch.int64, device=DEV)
    assert ops.argmax_merge_packed(packed, world, T, out).tolist() == [20, 30]


@pytest.mark.parametrize("nq,nkv,splits", [(8, 2, 1), (8, 8, 3), (4, 2, 4), (16, 2, 2)])
def test_paged_attention_decode(ops, nq, nkv, splits):
    D, bs, B = 128, 16, 5
    ctx = torch.tensor([1, 17, 100, 333, 64], dtype=torch.int32)
    max_blocks = (int(ctx.max()) + bs - 1) // bs
    nblocks = B * max_blocks + 3
    kc, vc = rnd(nblocks * bs, nkv, D, seed=16), rnd(nblocks * bs, nkv, D, seed=17)
    perm = torch.randperm(nblocks, generator=torch.Generator().manual_seed(1))
    bt = perm[: B * max_blocks].view(B, max_blocks).to(torch.int32)
    q = rnd(B, nq, D, seed=18)
    out = torch.empty_like(q)
    ws = ops.attn_workspace(B, nq, nkv, splits, DEV)
    scale = 1 / math.sqrt(D)
    for _ in range(2):
        ops.paged_attention(q, kc, vc, bt.to(DEV), ctx.to(DEV), out, scale, bs, splits=splits, workspace=ws)
    torch.cuda.synchronize()
    for b in range(B):
        rows = torch.cat([torch.arange(bs) + int(bt[b, j]) * bs for j in range(max_blocks)])[: int(ctx[b])].to(DEV)
        want = ref.attention(q[b: b + 1], kc[rows], vc[rows], scale)
        assert (out[b: b + 1].float() - want).abs().max().item() < 2e-2


def test_paged_attention_as_causal_prefill(ops):
    nq, nkv, D, bs, T = 8, 2, 128, 16, 70
    kc, vc = rnd(8 * bs, nkv, D, seed=19), rnd(8 * bs, nkv, D, seed=20)
    bt = torch.tensor([[3, 1, 6, 0, 2]], dtype=torch.int32, device=DEV)
    q = rnd(T, nq, D, seed=21)
    out = torch.empty_like(q)
    ctx = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    seqof = torch.zeros(T, dtype=torch.int32, device=DEV)
    ops.paged_attention(q, kc, vc, bt, ctx, out, 0.1, bs, seq_of_query=seqof)
    rows = torch.cat([torch.arange(bs) + int(b) * bs for b in bt[0]])[:T].to(DEV)
    want = ref.attention(q, kc[rows], vc[rows], 0.1, causal_offset=0)
    assert (out.float() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("T,nq,nkv,K,splits,bias", [(8, 8, 2, 512, 1, False), (5, 4, 4, 4096, 0, True), (70, 8, 2, 1024, 2, False),
                                                     (300, 2, 1, 256, 1, True), (16, 16, 4, 4096, 8, False)])
def test_qkv_gemm_with_rope_epilogue_equals_gemm_then_rope(ops, T, nq, nkv, K, splits, bias):
    D, bs = 128, 16
    M = (nq + 2 * nkv) * D
    x, w = rnd(T, K, seed=31), rnd(M, K, scale=0.05, seed=32)
    b = rnd(M, seed=33) if bias else None
    pos = (torch.arange(T, dtype=torch.int32) * 3 % 200).to(DEV)
    cs = ops.rope_cos_sin(D, 256, 5e5, DEV)
    nslots = bs * ((T + bs - 1) // bs + 2)
    slots = torch.randperm(nslots, generator=torch.Generator().manual_seed(2))[:T].to(DEV)
    slots[T // 2] = -1
    kc1, vc1 = torch.zeros(nslots, nkv, D, dtype=torch.bfloat16, device=DEV), torch.zeros(nslots, nkv, D, dtype=torch.bfloat16, device=DEV)
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    ref_qkv = ops.gemm(x, w, bias=b, splits=splits)
    ops.rope_kv(ref_qkv, pos, cs, slots, kc1, vc1, nq, nkv, D)
    got = torch.zeros(T, M, dtype=torch.bfloat16, device=DEV)
    ops.gemm_qkv_rope(x, w, got, pos, cs, slots, kc2, vc2, nq, nkv, bias=b, splits=splits)
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    assert torch.equal(got, ref_qkv) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)


@pytest.mark.parametrize("nq,nkv", [(8, 2), (8, 1), (4, 4), (4, 2)])
def test_prefill_attention_query_tiled(ops, nq, nkv):
    """Several sequences of different lengths in one batch of prompt rows, second chunk semantics
    included (rows whose context starts beyond 0 because earlier tokens are already cached)."""
    D, bs = 128, 16
    lens, starts = [70, 5, 33], [0, 40, 16]            # rows per sequence, tokens already in the cache
    nblocks = 40
    kc, vc = rnd(nblocks * bs, nkv, D, seed=41), rnd(nblocks * bs, nkv, D, seed=42)
    bt = torch.randperm(nblocks, generator=torch.Generator().manual_seed(3))[:27].view(3, 9).to(torch.int32)
    seqof = torch.tensor(sum(([s] * n for s, n in enumerate(lens)), []), dtype=torch.int32)
    ctx = torch.tensor(sum(([starts[s] + i + 1 for i in range(n)] for s, n in enumerate(lens)), []), dtype=torch.int32)
    T = int(seqof.numel())
    q = rnd(T, nq, D, seed=43)
    tiles = ops.prefill_tiles(seqof, nq // nkv)
    assert int(tiles[:, 1].sum()) == T and int(tiles[:, 1].max()) <= 64 // (nq // nkv)
    out = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, bt.to(DEV), ctx.to(DEV), seqof.to(DEV), tiles.to(DEV), out, 0.09, bs)
    torch.cuda.synchronize()
    want = torch.zeros_like(out)
    ops.paged_attention(q, kc, vc, bt.to(DEV), ctx.to(DEV), want, 0.09, bs, seq_of_query=seqof.to(DEV))   # one CTA per row
    r0 = 0
    for s, n in enumerate(lens):
        rows = torch.cat([torch.arange(bs) + int(b) * bs for b in bt[s]])[: starts[s] + n].to(DEV)
        ref_o = ref.attention(q[r0:r0 + n], kc[rows], vc[rows], 0.09, causal_offset=starts[s])
        assert (out[r0:r0 + n].float() - ref_o).abs().max().item() < 2e-2
        r0 += n
    assert (out.float() - want.float()).abs().max().item() < 2e-2


def test_gemm_announcing_the_next_weights_changes_nothing_but_timing():
    """ops.prefetch_next(w2) before a GEMM only asks for w2 to be brought into L2: same bits with and without, for the
    plain, the SiLU-mul and the QKV + RoPE kernels, with sizes that are no multiple of the prefetch chunk; an
    announcement holds for one launch."""
    from libtbvcoll_b200 import ops
    torch.manual_seed(7)
    x = (torch.randn(8, 4096, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(2048, 4096, device=DEV) * 0.02).to(torch.bfloat16)      # 16 MB: above the default "own weights" threshold
    big = torch.empty(100 * 1024 * 1024 + 4112, dtype=torch.uint8, device=DEV)      # more than the cap, odd tail
    nxt = [big, big[16:16 + 1000 * 16], torch.empty(24, dtype=torch.bfloat16, device=DEV), big[: 3 * 4096 + 16]]
    want = ops.gemm(x, w)
    for t in nxt:
        ops.prefetch_next(t)
        got = ops.gemm(x, w)
        assert torch.equal(got, want)
    wg = (torch.randn(2048, 4096, device=DEV) * 0.02).to(torch.bfloat16)
    want_g = ops.gemm(x, wg, epi=ops.EPI_SILU_MUL)
    ops.prefetch_next(big)
    assert torch.equal(ops.gemm(x, wg, epi=ops.EPI_SILU_MUL), want_g)
    assert torch.equal(ops.gemm(x, w), want)          # no announcement pending: the plain launch again
    torch.cuda.synchronize()
