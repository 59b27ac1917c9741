"""The stock-PyTorch baseline model (the oracle for the sm_100a engine) checked against itself:
tensor-parallel over gloo equals the single-rank model in fp32."""
from _workers import run_ranks, cpu_torch_baseline_tp
from conftest import free_port


def test_tp2_equals_tp1_fp32_over_gloo():
    res = run_ranks(cpu_torch_baseline_tp, 2, free_port(), timeout=240)
    for r in res:
        assert r["err"] <= 1e-4 * max(1.0, r["scale"])
        assert r["ars"] > 0
    assert res[0]["toks"] == res[1]["toks"] and len(res[0]["toks"][0]) == 4
