"""Build the native library in-tree with nvcc for sm_100a.

The reference has no build system, only a one-line hipcc command (README.md:6-7,
step4/libtbvcoll.cpp:27).  Here every translation unit under ``csrc/`` is compiled
with ``-gencode arch=compute_100a,code=sm_100a`` and linked into ONE shared object,
``libtbvcoll_b200/libtbvcoll.so``, which exports the collective ABI (``tbv_ar_*``,
``tbv_comm_*``) and the operator ABI (``tbv_op_*``).  Objects are rebuilt only when a
source or header is newer.

    python -m libtbvcoll_b200._build [--force] [--verbose] [--bounds]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libtbvcoll.so"
LIB_BOUNDS = PKG / "libtbvcoll_bounds.so"     # the same sources with -DTBV_BOUNDS_CHECK (device-side extent guards)
AR_BENCH = PKG / "tbv_arbench"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
          "--expt-relaxed-constexpr", "-I", str(CSRC)]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the native library cannot be built")
    return exe


def lib_sources() -> list[Path]:
    srcs = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp")) + sorted((CSRC / "ops").glob("*.cu"))
    return srcs


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((CSRC / "ops").glob("*.cuh")) + list((CSRC / "ops").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, force: bool, verbose: bool, hdr_m: float, bounds: bool = False) -> tuple[Path, str]:
    obj = (OBJ / "bounds" if bounds else OBJ) / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_m):
        return obj, ""
    cmd = [nvcc(), *ARCH, *COMMON, *(["-DTBV_BOUNDS_CHECK"] if bounds else []), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{p.stdout}\n{p.stderr}")
    return obj, p.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link; returns the path of the shared object."""
    OBJ.mkdir(exist_ok=True)
    srcs = lib_sources()
    hdr_m = _headers_mtime()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose, hdr_m), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log, file=sys.stderr)
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        _link(LIB, objs)
    # standalone microbenchmark executable (counterpart of the reference's ar2/armr binaries)
    proto = CSRC / "proto" / "arbench.cu"
    if proto.exists() and (force or not AR_BENCH.exists() or AR_BENCH.stat().st_mtime < max(proto.stat().st_mtime, LIB.stat().st_mtime)):
        cmd = [nvcc(), *ARCH, *COMMON, str(proto), "-o", str(AR_BENCH), f"-L{PKG}", "-ltbvcoll",
               "-Xlinker", "-rpath,$ORIGIN"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"arbench build failed:\n{p.stdout}\n{p.stderr}")
    return LIB


def _link(target: Path, objs) -> None:
    """Link under a temporary name and rename into place: a reader (a process that has the library mapped, a copy
    of the tree being taken) sees the old file or the new one, never a half-written one."""
    tmp = target.with_name(target.name + f".tmp{os.getpid()}")
    cmd = [nvcc(), *ARCH, "-shared", "-o", str(tmp), *map(str, objs), "-lrt", "-lpthread", "-ldl"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"link failed:\n{p.stdout}\n{p.stderr}")
    os.replace(tmp, target)


def build_bounds(force: bool = False) -> Path:
    """The bounds-checked debug library, ``libtbvcoll_bounds.so`` (load it with ``TBV_LIB=<path>``).
    compute-sanitizer's stand-in for the collective kernels: see ``TBV_GUARD`` in csrc/ar_device.cuh."""
    (OBJ / "bounds").mkdir(parents=True, exist_ok=True)
    srcs = lib_sources()
    hdr_m = _headers_mtime()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = [o for o, _ in ex.map(lambda s: _compile(s, force, False, hdr_m, bounds=True), srcs)]
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB_BOUNDS.exists() or LIB_BOUNDS.stat().st_mtime < newest:
        _link(LIB_BOUNDS, objs)
    return LIB_BOUNDS


def ensure_built() -> Path:
    """Build if the shared object is missing or stale (cheap mtime check)."""
    try:
        srcs = lib_sources()
        newest = max([s.stat().st_mtime for s in srcs] + [_headers_mtime()])
        if LIB.exists() and LIB.stat().st_mtime >= newest:
            return LIB
    except OSError:
        if LIB.exists():
            return LIB
    return build()


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(out)
    if "--bounds" in sys.argv:
        print(build_bounds(force="--force" in sys.argv))
