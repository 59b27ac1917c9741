"""Real multi-GPU ranks, one process per GPU (skipped when the box has a single GPU).
Run with 2 or more GPUs visible, e.g. ``pytest tests/test_multigpu.py -m gpu``."""
import pytest
import torch

from _workers import run_ranks, gpu_collectives, gpu_engine_tp, gpu_peer_skips, gpu_fused_gemm_ar, gpu_sp_kernels, gpu_stream_wait_mode
from conftest import free_port

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worlds():
    """World sizes to exercise: every power of two the box can host, or TBV_TEST_WORLDS=8 (comma list)."""
    import os
    only = os.environ.get("TBV_TEST_WORLDS")
    ws = [int(x) for x in only.split(",")] if only else [2, 4, 8]
    return [w for w in ws if w <= NGPU]


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("mem", ["vmm", "ipc"])
def test_collectives_exact_stress_graph_fused(mem):
    for world in _worlds():
        res = run_ranks(gpu_collectives, world, free_port(), mem, timeout=300)
        for r in res:
            assert r["bad"] == [] and r["stress_bad"] == 0
            assert r["graph_ok"] and r["fused_ok"] and r["rs_ok"] and r["ag_ok"]
            assert r["over_cap"] is False and not r["err"]
            assert r["stats"][5] > 0


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
def test_engine_tensor_parallel():
    for world in _worlds():
        res = run_ranks(gpu_engine_tp, world, free_port(), timeout=300)
        assert len({r["hash"] for r in res}) == 1
        for r in res:
            assert r["loops_equal"] and r["fallbacks"] == 0
            assert r["sp_equals_allreduce_path"]
            assert r["sp_chunks"] > 0 or world > 4      # the 64-row test chunks do not divide into 8 x 16 rows
            assert r["fused_gemm_token_agreement"] == 1.0     # one kernel or two: identical bits, identical tokens
            assert r["logit_err"] < 0.05 * r["logit_scale"] + 0.02


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
def test_peer_drops_a_call_device_watchdog():
    res = run_ranks(gpu_peer_skips, 2, free_port(), timeout=120)
    r0 = res[0]
    assert r0["first"] == 2.0 and r0["err"] and r0["refused"] and r0["alive"] == 16.0
    assert 0.4 < r0["elapsed"] < 10
    assert r0["last"]["code"] == 1 and r0["last"]["peer"] == 1


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
def test_stream_wait_value_mode_real_ranks():
    res = run_ranks(gpu_stream_wait_mode, 2, free_port(), timeout=120)
    assert all(r["bad"] == [] and not r["err_before"] for r in res)
    r0 = res[0]
    assert r0["failed"] and r0["err"] and r0["alive"] == 16.0 and 0.4 < r0["elapsed"] < 10
    assert r0["last"]["code"] == 1 and r0["last"]["peer"] == 1 and r0["last"]["where"] == 4


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
def test_fused_gemm_allreduce_rmsnorm_real_ranks():
    for world in _worlds():
        res = run_ranks(gpu_fused_gemm_ar, world, free_port(), timeout=300)
        assert all(r["ok"] and not r["err"] for r in res)
        assert all(r["hashes"] == res[0]["hashes"] for r in res)      # identical bits on every rank


@pytest.mark.skipif(NGPU < 2, reason="needs >= 2 GPUs")
def test_sequence_parallel_kernel_pairs_real_ranks():
    for world in _worlds():
        res = run_ranks(gpu_sp_kernels, world, free_port(), timeout=300)
        assert all(r["ok"] and not r["err"] for r in res)
