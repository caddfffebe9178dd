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


def build(force: bool = False, verbose: bool = False, lib_path: Path = None, extra_flags=()) -> Path:
    """Builds what is out of date.  ``lib_path`` / ``extra_flags`` make a variant of the library somewhere else (its
    objects live beside it), e.g. ``-DTPB_GEMM_TRACE`` for the kernel-internal phase trace or ``-DTPB_BOUNDS`` for the
    in-kernel bounds checks; ``TPB_LIB_PATH`` makes ``ops.native`` load such a variant."""
    nvcc = _nvcc()
    lib_path = Path(lib_path) if lib_path is not None else LIB_PATH
    obj_dir = OBJ_DIR if lib_path == LIB_PATH else lib_path.parent / (lib_path.stem + "_obj")
    obj_dir.mkdir(parents=True, exist_ok=True)
    lib_path.parent.mkdir(parents=True, exist_ok=True)
    header_time = _newest_header_mtime()
    flags = list(NVCC_FLAGS) + list(extra_flags) + os.environ.get("TPB_NVCC_FLAGS", "").split()
    jobs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
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
    objs = [str(obj_dir / (src.stem + ".o")) for src in sources()]
    newest_obj = max(os.path.getmtime(o) for o in objs)
    if force or jobs or not lib_path.exists() or lib_path.stat().st_mtime < newest_obj:
        run([nvcc, "-shared", "-o", str(lib_path), *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
