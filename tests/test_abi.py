"""The exported C ABI and the Python module surface keep the reference's names
(step4/libtbvcoll.cpp:279-566, step4/tbvcoll.py:14-111)."""
import ctypes


def test_reference_symbols_are_exported():
    from libtbvcoll_b200.tbvcoll import load_library
    l = load_library()
    for name in ("tbv_ar_init", "tbv_ar_allreduce", "tbv_ar_stats", "tbv_ar_stats4", "tbv_ar_stats5", "tbv_ar_cap", "tbv_ar_async",
                 "tbv_ar_err", "tbv_ar_rails", "tbv_ar_hist", "tbv_ar_fini",
                 # additions of this build
                 "tbv_ar_init_n", "tbv_ar_cap64", "tbv_ar_sync", "tbv_comm_create", "tbv_comm_create_local", "tbv_comm_allreduce",
                 "tbv_comm_allreduce_rmsnorm", "tbv_comm_gemm_allreduce_rmsnorm", "tbv_comm_gemm_reduce_scatter",
                 "tbv_comm_allgather_gemm", "tbv_comm_reduce_scatter", "tbv_comm_all_gather", "tbv_op_gemm", "tbv_op_gemm_qkv_rope",
                 "tbv_op_paged_attention", "tbv_op_prefill_attention", "tbv_op_rmsnorm", "tbv_op_argmax", "tbv_op_argmax_noalloc",
                 "tbv_comm_trace", "tbv_comm_timestamps", "tbv_comm_mute_rank", "tbv_comm_tag_counts", "tbv_op_gemm_prefetch_next",
                 "tbv_op_copy_async"):
        assert isinstance(getattr(l, name), ctypes._CFuncPtr), name


def test_python_module_surface_and_uninitialised_contract():
    import torch
    import tbvcoll          # the reference's module name
    for fn in ("init", "all_reduce", "is_async", "err", "rails", "hist", "raw_fn", "cap", "stats5", "stats4", "stats3", "stats"):
        assert callable(getattr(tbvcoll, fn)), fn
    from libtbvcoll_b200 import tbvcoll as t
    if not t._ready:
        assert t.all_reduce(torch.ones(4)) is False          # not initialised -> caller falls back


def test_cap_is_rounded_to_4k_and_knob_clamps(monkeypatch):
    """cap rounds up to 4 KiB (reference: libtbvcoll.cpp:281); TBV_NSLOT clamps to 2..32 (:287-288)."""
    from libtbvcoll_b200.tbvcoll import Comm
    monkeypatch.setenv("TBV_NSLOT", "1")
    c = Comm(0, 1, -1, "127.0.0.1", 0, cap_bytes=5000)       # world 1 on the CPU backend: no peers needed
    try:
        assert c.cap == 8192 and c.nslot() == 2
        x = torch_ones()
        assert c.all_reduce(x) and x[0].item() == 1.0        # world 1: identity
    finally:
        c.destroy()


def torch_ones():
    import torch
    return torch.ones(8)
