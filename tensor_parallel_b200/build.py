"""Build of the native library ``tensor_parallel_b200/lib/libtpb200.so`` (sm_100a only).

Every ``csrc/*.cu`` is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` to an object
file (in parallel) and linked into one shared library with a C ABI, loaded through ``ctypes``.
nvcc cross-compiles without a GPU, so the library can be built on a CPU-only machine and shipped.
``python -m tensor_parallel_b200.build`` rebuilds what is out of date.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libtpb200.so"
OBJ_DIR = PKG / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    header_time = _newest_header_mtime()
    flags = list(NVCC_FLAGS) + os.environ.get("TPB_NVCC_FLAGS", "").split()  # e.g. -DTPB_GEMM_TRACE, -DTPB_BOUNDS
    jobs = []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time)
        if stale:
            jobs.append([nvcc, *flags, *( ["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)])

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        return proc.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for log in pool.map(run, jobs):
                if verbose and log:
                    print(log, file=sys.stderr)
    objs = [str(OBJ_DIR / (src.stem + ".o")) for src in sources()]
    newest_obj = max(os.path.getmtime(o) for o in objs)
    if force or jobs or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        run([nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
