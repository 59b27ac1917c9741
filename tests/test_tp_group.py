"""TPGroup on the CPU backend: calls the library takes are counted as launches, calls it declines
(over capacity, non-contiguous) go to torch.distributed and are counted as fallbacks — the hook's
behaviour in the reference (step3b/vllm_tp_bench.py:108-124)."""
from _workers import run_ranks, cpu_tp_group_fallback
from conftest import free_port


def test_tp_group_counts_and_falls_back_over_gloo():
    res = run_ranks(cpu_tp_group_fallback, 2, free_port(), free_port(), timeout=180)
    for r in res:
        assert all(r["ok"]), r
        assert r["calls"] == 5 and r["fallbacks"] == 2 and r["launches"] == 3


def test_world_one_is_a_pass_through():
    import torch
    from libtbvcoll_b200.parallel.tp import TPGroup
    tp = TPGroup()
    x = torch.arange(8.0)
    assert tp.all_reduce(x) is x and tp.calls == 0
    out = torch.empty(8)
    assert torch.equal(tp.all_gather(x, out), x) and torch.equal(tp.reduce_scatter(x, torch.empty(8)), x)
