"""Text patches on an installed vLLM, kept for parity with the reference's step3b/dbo_patch.py.

The reference rewrote three vLLM source files to get past the assertions that block dual-batch
overlap (DBO) with DP=1 (dbo_patch.py:19-65), showed that the resulting overlap was a no-op and
withdrew DBO as a goal (reports/11_custom_engine.md:121-151, reports/12_references.md:49-65).
This module keeps the mechanism — ``patch(module, needle, repl, label)`` rewrites a module's
source file once, idempotently, with a backup — and a ``survey()`` that reports which of the
reference's needles exist in the installed vLLM, so a user can see why nothing is patched by
default.  In this library communication/compute overlap comes from programmatic dependent launch
and GEMM-epilogue fusion, not from DBO.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
from typing import Dict, Optional

NEEDLES = {
    "config all2all assert": ("vllm.config.parallel", "all2all"),
    "SM control only on CUDA": ("vllm.v1.worker.ubatching", "current_platform.is_cuda()"),
    "should_ubatch gate": ("vllm.v1.worker.ubatch_utils", "should_ubatch"),
}


def _source_of(module: str) -> Optional[str]:
    try:
        spec = importlib.util.find_spec(module)
    except (ImportError, ValueError):
        return None
    return spec.origin if spec and spec.origin and spec.origin.endswith(".py") else None


def patch(module: str, needle: str, repl: str, label: str, dry_run: bool = False) -> bool:
    """Replace the first occurrence of ``needle`` in ``module``'s source by ``repl``.  Returns True
    if the file now contains ``repl`` (patched now or earlier).  A ``.tbv-orig`` backup is kept."""
    path = _source_of(module)
    if path is None:
        print(f"[dbo_patch] {label}: module {module} not found")
        return False
    src = open(path).read()
    if repl in src:
        return True
    if needle not in src:
        print(f"[dbo_patch] {label}: needle not found in {path} (different vLLM version)")
        return False
    if dry_run:
        return True
    if not os.path.exists(path + ".tbv-orig"):
        shutil.copy2(path, path + ".tbv-orig")
    with open(path, "w") as f:
        f.write(src.replace(needle, repl, 1))
    print(f"[dbo_patch] {label}: patched {path}")
    return True


def unpatch(module: str) -> bool:
    path = _source_of(module)
    if path and os.path.exists(path + ".tbv-orig"):
        shutil.move(path + ".tbv-orig", path)
        return True
    return False


def survey() -> Dict[str, bool]:
    """Which of the reference's patch sites exist in the installed vLLM."""
    out = {}
    for label, (module, needle) in NEEDLES.items():
        path = _source_of(module)
        out[label] = bool(path) and needle in open(path).read()
    return out


if __name__ == "__main__":
    for k, v in survey().items():
        print(f"{k}: {'present' if v else 'absent'}")
