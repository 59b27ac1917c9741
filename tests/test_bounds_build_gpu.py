"""The bounds-checked debug build (``python -m libtbvcoll_b200._build --bounds``): the stand-in for
compute-sanitizer on hosts where that tool is not available.  The same sources compiled with
-DTBV_BOUNDS_CHECK compare, inside every collective kernel, the extent about to be touched with what the
communicator reserved.  Checked here in a child process that loads that library (TBV_LIB):
  * results are still exact;
  * a violation — made harmlessly by telling the guards (TBV_DEBUG_CAP) that less is reserved than really
    is, so the call stays inside real memory — is recorded with its site and the offending extent, no data
    is moved, the error is sticky, the kernel ends and the context stays usable."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import torch
from libtbvcoll_b200.tbvcoll import Comm, load_library
assert load_library().tbv_bounds_checked_build() == 1
world = 4
c = Comm.local(world, 0, cap_bytes=1 << 16)
def gen(seed, n):
    return ((torch.rand(n, generator=torch.Generator().manual_seed(seed)) - 0.5) * 10).to(torch.bfloat16).cuda()
def oracle(ts):
    acc = ts[0].float()
    for t in ts[1:]:
        acc = acc + t.float()
    return acc.to(ts[0].dtype)
for algo in ("oneshot", "ll", "twoshot"):           # inside the guarded extent: exact as ever
    c.set_algo(algo)
    ins = [gen(10 + r, 1024) for r in range(world)]
    outs = [torch.empty_like(t) for t in ins]
    assert c.all_reduce_local(ins, outs)
    torch.cuda.synchronize()
    assert all(torch.equal(o, oracle(ins)) for o in outs), algo
assert not c.err()
c.set_algo("oneshot")
ins = [gen(50 + r, 4096) for r in range(world)]     # 8192 bytes > the 4096 the guards were told about
outs = [torch.full_like(t, 7.0) for t in ins]
assert c.all_reduce_local(ins, outs)
torch.cuda.synchronize()                            # the kernel ends
assert c.err()
last = c.last_error()
assert last["code"] == 3 and last["where"] == 16 and last["seq"] == 8192, last
assert all(bool((o == 7.0).all()) for o in outs)    # nothing was moved
try:
    c.all_reduce_local(ins, outs)
    raise SystemExit("a call after the violation was accepted")
except RuntimeError:
    pass
assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
c.destroy()
print("BOUNDS-OK")
"""


def test_bounds_checked_build_is_exact_and_records_violations():
    from libtbvcoll_b200 import _build
    from libtbvcoll_b200.tbvcoll import load_library
    assert load_library().tbv_bounds_checked_build() == 0          # the normal build carries no guards
    lib = _build.build_bounds()
    env = dict(os.environ, TBV_LIB=str(lib), TBV_DEBUG_CAP="4096")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-c", CHILD], env=env, cwd=root, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0 and "BOUNDS-OK" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
