"""Ahead-of-time build of the CUDA library (sm_100a only).

Usage: ``python -m flashrnn_b200.build``. The shared object is written next to the package
(``flashrnn_b200/lib/libflashrnn_b200.so``) so that it travels with the source tree; nothing is
JIT-compiled at import time (the reference compiles per shape at first use,
flashrnn/flashrnn/cuda_init.py:139-168).
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libflashrnn_b200.so"
SOURCES = ("capi.cu", "capi_mg.cu", "recurrent_fwd.cu", "recurrent_fwd_ksplit.cu", "recurrent_bwd.cu", "recurrent_bwd_ksplit.cu",
           "recurrent_mg_fwd.cu", "recurrent_mg_bwd.cu", "wgrad.cu", "input_proj.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
)


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + [src, PKG.parent / "include" / "flashrnn_b200.h"])
    return obj.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every translation unit (in parallel) and link the shared library."""
    nvcc = _nvcc()
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = [s for s in SOURCES if (CSRC / s).exists()]
    jobs = []
    for name in sources:
        src, obj = CSRC / name, obj_dir / (name + ".o")
        if force or _stale(obj, src):
            jobs.append([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)])

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        if verbose and res.stderr:
            print(res.stderr, file=sys.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        list(pool.map(run, jobs))
    objs = [str(obj_dir / (s + ".o")) for s in sources]
    if jobs or not LIB_PATH.exists():
        # link next to the target, then rename: a reader (or a copy of the tree) never sees a half-written library
        tmp = LIB_PATH.with_suffix(".so.tmp")
        run([nvcc, "-shared", "-o", str(tmp), *objs])
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
