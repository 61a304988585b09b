"""ctypes loader for ``oracle/cpu_gemm.c`` (test infrastructure, parity unpinned).

The C file states the numeric contract; this module only builds it (``make``),
loads it and wraps the calls in numpy arrays of ``uint16`` (raw bf16 bits).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

__all__ = [
    "build", "lib", "fill_bf16", "gemm_bf16", "gemm_f32out", "gemm_naive", "check",
    "max_abs_bf16", "num_threads", "set_num_threads", "host_cores", "bf16_to_f32", "f32_to_bf16", "NORMAL", "UNIFORM",
]

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "liboracle.so"
_lib = None

NORMAL = 0
UNIFORM = 1


def build(force: bool = False) -> Path:
    """Compile cpu_gemm.c with gcc + OpenMP if the library is missing or stale."""
    src = _HERE / "cpu_gemm.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(_HERE)] + (["-B"] if force else []), check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_SO))
        u16p = ctypes.POINTER(ctypes.c_uint16)
        f32p = ctypes.POINTER(ctypes.c_float)
        L.maize_oracle_fill_bf16.argtypes = [ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_double,
                                             ctypes.c_uint64, ctypes.c_uint64, u16p]
        L.maize_oracle_fill_bf16.restype = None
        L.maize_oracle_gemm_bf16.argtypes = [u16p, ctypes.c_uint32, ctypes.c_uint32, u16p, ctypes.c_uint32,
                                             ctypes.c_uint32, u16p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int]
        L.maize_oracle_gemm_bf16.restype = ctypes.c_int
        L.maize_oracle_gemm_bf16_ld.argtypes = [u16p, ctypes.c_uint64, u16p, ctypes.c_uint64, u16p, ctypes.c_uint64,
                                                ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int]
        L.maize_oracle_gemm_bf16_ld.restype = ctypes.c_int
        L.maize_oracle_gemm_f32out.argtypes = [u16p, u16p, f32p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                               ctypes.c_int]
        L.maize_oracle_gemm_f32out.restype = ctypes.c_int
        L.maize_oracle_gemm_naive.argtypes = [u16p, u16p, u16p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]
        L.maize_oracle_gemm_naive.restype = None
        L.maize_oracle_check.argtypes = [u16p, ctypes.c_uint64, u16p, ctypes.c_uint64, ctypes.c_uint32,
                                         ctypes.c_uint32, ctypes.c_uint32, ctypes.c_double, ctypes.c_double,
                                         ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_uint64)]
        L.maize_oracle_check.restype = ctypes.c_int
        L.maize_oracle_max_abs_bf16.argtypes = [u16p, ctypes.c_uint64]
        L.maize_oracle_max_abs_bf16.restype = ctypes.c_double
        L.maize_oracle_num_threads.restype = ctypes.c_int
        L.maize_oracle_set_num_threads.argtypes = [ctypes.c_int]
        L.maize_oracle_set_num_threads.restype = None
        L.maize_oracle_f32_to_bf16.argtypes = [ctypes.c_float]
        L.maize_oracle_f32_to_bf16.restype = ctypes.c_uint16
        L.maize_oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.maize_oracle_bf16_to_f32.restype = ctypes.c_float
        _lib = L
    return _lib


def _u16(a: np.ndarray):
    assert a.dtype == np.uint16 and a.flags.c_contiguous
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))


def num_threads() -> int:
    return int(lib().maize_oracle_num_threads())


def set_num_threads(n: int) -> None:
    """Thread count of every later call (overrides an inherited OMP_NUM_THREADS)."""
    lib().maize_oracle_set_num_threads(int(n))


def host_cores() -> int:
    """Cores this process may run on (its affinity mask), not what OMP_NUM_THREADS says."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def fill_bf16(seed: int, matrix_id: int, shape, dist: int = NORMAL, scale: float = 1.0, first: int = 0) -> np.ndarray:
    """Seeded bf16 matrix (raw bits, uint16).  matrix_id: 0 = A, 1 = B."""
    out = np.empty(shape, dtype=np.uint16)
    lib().maize_oracle_fill_bf16(seed, matrix_id, dist, float(scale), first, out.size, _u16(out))
    return out


def gemm_bf16(a: np.ndarray, b: np.ndarray, nthreads: int = 0) -> np.ndarray:
    """C = A @ B.T on raw bf16 bits: fp32 ascending-k sum, one RNE rounding."""
    M, K = a.shape
    N, Kb = b.shape
    c = np.empty((M, N), dtype=np.uint16)
    rc = lib().maize_oracle_gemm_bf16(_u16(a), M, K, _u16(b), N, Kb, _u16(c), M, N, nthreads)
    if rc != 0:
        raise ValueError("oracle: bad GEMM arguments (a_cols != b_cols?)")
    return c


def gemm_f32out(a: np.ndarray, b: np.ndarray, nthreads: int = 0) -> np.ndarray:
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb
    c = np.empty((M, N), dtype=np.float32)
    rc = lib().maize_oracle_gemm_f32out(_u16(a), _u16(b), c.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), M, N, K,
                                        nthreads)
    assert rc == 0
    return c


def gemm_naive(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    M, K = a.shape
    N, _ = b.shape
    c = np.empty((M, N), dtype=np.uint16)
    lib().maize_oracle_gemm_naive(_u16(a), _u16(b), _u16(c), M, N, K)
    return c


def max_abs_bf16(x: np.ndarray) -> float:
    x = np.ascontiguousarray(x)
    return float(lib().maize_oracle_max_abs_bf16(_u16(x), x.size))


def check(c: np.ndarray, ref: np.ndarray, K: int, max_abs_a: float, max_abs_b: float):
    """Return (ok, max_abs_err, bound, violations) for the path's tolerance."""
    assert c.shape == ref.shape
    M, N = c.shape
    c = np.ascontiguousarray(c)
    ref = np.ascontiguousarray(ref)
    err = ctypes.c_double()
    bound = ctypes.c_double()
    bad = ctypes.c_uint64()
    rc = lib().maize_oracle_check(_u16(c), N, _u16(ref), N, M, N, K, max_abs_a, max_abs_b, ctypes.byref(err),
                                  ctypes.byref(bound), ctypes.byref(bad))
    return rc == 0, err.value, bound.value, bad.value


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (x.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)


if __name__ == "__main__":
    print(build(force=bool(os.environ.get("FORCE"))))
