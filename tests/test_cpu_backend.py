"""CPU (shared-memory) backend: protocol, contract and host-side fault handling; no GPU.

Plays the role of the reference's two-node scripts test_exact.py / test_stress.py
(step4/test_exact.py:15-38, step4/test_stress.py:17-42) with both ranks as processes on
one host: inputs are regenerated from seeds on every rank and the oracle is a fixed-order
fp32 accumulation, never another collective library."""
import pytest

from _workers import run_ranks, cpu_async_stream, cpu_contract, cpu_rs_ag, cpu_peer_skips, cpu_never_joins
from conftest import free_port


def test_two_rank_bf16_1000_async_calls_4_slots():
    res = run_ranks(cpu_async_stream, 2, free_port(), 1000, 4, "bfloat16", (16, 4096), timeout=300)
    assert all(r["bad"] == 0 for r in res)
    assert res[0]["hash"] == res[1]["hash"]          # identical bits on both ranks
    assert all(r["n"] == 1000 for r in res)


@pytest.mark.parametrize("world,dtype", [(4, "float32"), (3, "float16"), (8, "bfloat16")])
def test_n_ranks_exact(world, dtype):
    res = run_ranks(cpu_async_stream, world, free_port(), 40, 2, dtype, (5, 129), timeout=300)
    assert all(r["bad"] == 0 for r in res)
    assert len({r["hash"] for r in res}) == 1


def test_contract():
    res = run_ranks(cpu_contract, 2, free_port())
    for r in res:
        assert r["cap"] == 8192
        assert r["zero"] is True
        assert r["big"] is False and r["int"] is False and r["noncontig"] is False and r["badout"] is False
        assert r["inplace"] is True and r["val"] == [3.0] * 7
        assert r["torch.float16"] and r["torch.bfloat16"] and r["torch.float32"]
        assert r["raw"] == (0, 4.0)
        assert r["raw_big"] == -2
        assert r["err"] is False


def test_reduce_scatter_all_gather():
    for ok_rs, ok_ag in run_ranks(cpu_rs_ag, 4, free_port()):
        assert ok_rs and ok_ag


def test_peer_drops_a_call_watchdog_fires_and_error_is_sticky():
    res = run_ranks(cpu_peer_skips, 2, free_port())
    r0 = res[0]
    assert r0["first"] == 2.0
    assert r0["failed"] and r0["err"] and r0["refused"]
    assert 0.25 < r0["elapsed"] < 5.0
    assert r0["last"]["peer"] == 1


def test_peer_never_joins_init_times_out():
    res = run_ranks(cpu_never_joins, 1, free_port())
    assert res[0]["raised"] and res[0]["elapsed"] < 10
