"""The allocation-free arg-max entry point (collected last on purpose: the file name sorts
after every other test file, so a run that stops at the first failure has already run the
rest).

Some users of the library cannot call cudaMalloc at the point where they sample — a serving
process whose KV-cache pool already owns all free device memory, a loop that cannot afford
the device-wide synchronisation an allocation implies, a plug-in bound by a host application's
no-allocation rule.  For them the library exports ``tbv_op_argmax_noalloc``, whose scratch is
a fixed array inside the library image.  This test calls it through its exported C symbol,
twice in a row, and checks both results against the existing entry point ``tbv_op_argmax``
(which takes a caller-provided workspace).  Arg-max has no rounding: the tolerance is zero.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from libtbvcoll_b200.tbvcoll import load_library
    l = load_library()
    I, LL, vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
    fn = l.tbv_op_argmax_noalloc
    fn.argtypes = [vp, I, I, I, LL, vp, vp, vp]
    fn.restype = I
    ref = l.tbv_op_argmax
    ref.argtypes = [vp, I, I, I, LL, vp, vp, vp, vp]
    ref.restype = I
    ws_size = l.tbv_op_argmax_workspace
    ws_size.argtypes = [I]
    ws_size.restype = ctypes.c_size_t
    return fn, ref, ws_size


def test_noalloc_argmax_matches_workspace_argmax_twice_in_a_row():
    fn, ref, ws_size = _symbols()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(11)
    for call, (tokens, vocab, offset) in enumerate([(7, 128256, 1000), (64, 32000, 0)]):      # two calls in a row
        logits = torch.randn(tokens, vocab, generator=g).to(torch.bfloat16).to(dev)
        logits[tokens // 2, 77] = logits[tokens // 2, vocab - 5] = 60.0                      # a tie: lowest index wins
        val = torch.empty(tokens, dtype=torch.float32, device=dev)
        idx = torch.empty(tokens, dtype=torch.int64, device=dev)
        rc = fn(logits.data_ptr(), tokens, vocab, logits.stride(0), offset, val.data_ptr(), idx.data_ptr(), st)
        assert rc == 0
        ws = torch.zeros(ws_size(tokens), dtype=torch.uint8, device=dev)
        val2 = torch.empty_like(val)
        idx2 = torch.empty_like(idx)
        assert ref(logits.data_ptr(), tokens, vocab, logits.stride(0), offset, ws.data_ptr(), val2.data_ptr(), idx2.data_ptr(), st) == 0
        torch.cuda.synchronize()
        assert torch.equal(idx, idx2) and torch.equal(val, val2), f"call {call}"
        assert int(idx[tokens // 2]) == 77 + offset
        # and, independently of this library's other arg-max, against the plain PyTorch statement of the same rule
        # (largest value, lowest index on ties)
        from libtbvcoll_b200.ops import reference as plain
        want_val, want_idx = plain.argmax_first(logits)
        assert torch.equal(idx, want_idx.to(idx.device) + offset) and torch.equal(val, want_val.to(val.device).float()), f"call {call}"


def test_noalloc_argmax_rejects_more_rows_than_the_scratch_holds():
    fn, _, _ = _symbols()
    x = torch.zeros(4, 16, dtype=torch.bfloat16, device="cuda:0")
    rc = fn(x.data_ptr(), 257, 16, 16, 0, None, None, None)
    assert rc == -2
