"""Builds ``maize_b200/_lib/libmaize_gemm.so`` from ``csrc/`` with nvcc for sm_100a.

Run as ``python -m maize_b200.build``.  nvcc cross-compiles without a GPU; the
library links the CUDA runtime statically and resolves the one driver symbol it
needs (``cuTensorMapEncodeTiled``) at run time, so it loads on a machine with
no driver and reports ``MAIZE_ERR_NO_DEVICE`` there instead of failing to load.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_lib" / "libmaize_gemm.so"
SOURCES = [CSRC / "maize_gemm.cu", CSRC / "maize_mgpu.cu"]
DEPENDS = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "maize_gemm.h"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-shared", "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return nvcc


def is_stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    return any(d.stat().st_mtime > t for d in DEPENDS if d.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return OUT
    OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(OUT), *map(str, SOURCES)]
    env = dict(os.environ)
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libmaize_gemm.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
