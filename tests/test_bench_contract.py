"""bench.py's command line contract that can be checked without a GPU: the reference arm answers with one
JSON line and exit code 0 (the reference is HIP + Thunderbolt ibverbs and cannot be installed or run here)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_unavailable_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-500:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]


def test_help_lists_the_driver_flags():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in r.stdout


def test_phase_stats_of_a_synthetic_trace():
    """The cross-rank arithmetic behind ``bench_allreduce --trace``: two ranks with timers 1 s apart, rank 1 always pushes
    0.5 us later than rank 0; flight is 2 us.  Each rank sees the other's payload 2 us after that rank's push."""
    import torch
    from libtbvcoll_b200.bench_allreduce import phase_stats
    calls, period = 6, 10_000
    rows = []
    for r, (offset, push_at) in enumerate([(0, 1_000), (1_000_000_000, 1_500)]):
        other_push = 1_500 if r == 0 else 1_000
        rr = []
        for k in range(calls):
            t0 = offset + k * period
            ready = t0 + max(push_at, other_push + 2_000)
            rr.append([k + 1, t0, t0 + push_at, ready, ready + 700])
        rows.append(rr)
    st = phase_stats(torch.tensor(rows, dtype=torch.int64))
    assert st["calls"] == calls and st["calls_with_push_stamp"] == calls
    assert st["push_issue"] == 1.25                                   # (1.0 + 1.5) / 2
    assert st["wait_after_push_least_waiting_rank"] == 1.5            # rank 1: sees rank 0's payload at 3.0, pushed at 1.5
    assert st["wait_after_push_most_waiting_rank"] == 2.5             # rank 0: sees rank 1's payload at 3.5, pushed at 1.0
    assert st["reduce_store_done"] == 0.7 and st["period_median"] == 10.0
    rows[1][2][0] = 99                                                # ranks that hold different calls cannot be aligned
    assert phase_stats(torch.tensor(rows, dtype=torch.int64)) is None
    rows[1][2][0] = 3
    rows[0][4][2] = 0                                                 # a call whose kernel takes no push stamp is left out of the push figures
    st = phase_stats(torch.tensor(rows, dtype=torch.int64))
    assert st["calls_with_push_stamp"] == calls - 1 and st["push_issue"] == 1.25
