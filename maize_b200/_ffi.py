"""ctypes binding of the C ABI in ``include/maize_gemm.h``.

The shared library is the product; there is no Python or CPU fallback.  A
missing library raises ``ImportError`` with the build command, and a missing
GPU surfaces as ``MaizeError(NO_DEVICE)`` from ``Context()``.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libmaize_gemm.so"

OK, INVALID_ARG, UNSUPPORTED, CUDA, TIMEOUT, DEVICE_ABORT, NO_DEVICE = range(7)
STATUS_NAMES = {
    OK: "MAIZE_OK", INVALID_ARG: "MAIZE_ERR_INVALID_ARG", UNSUPPORTED: "MAIZE_ERR_UNSUPPORTED",
    CUDA: "MAIZE_ERR_CUDA", TIMEOUT: "MAIZE_ERR_TIMEOUT", DEVICE_ABORT: "MAIZE_ERR_DEVICE_ABORT",
    NO_DEVICE: "MAIZE_ERR_NO_DEVICE",
}

# Every symbol include/maize_gemm.h declares: (restype, argtypes)
_vp, _u32, _u64, _i64, _int = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int


class GlobalMatrix(ctypes.Structure):
    """``maize_global_matrix_t``: {ptr, nrows, ncols}, the reference's GlobalMatrix (src/main.rs:20-27)."""
    _fields_ = [("ptr", _vp), ("nrows", _u32), ("ncols", _u32)]


_gm = ctypes.POINTER(GlobalMatrix)
SYMBOLS = {
    "maize_version": (_int, []),
    "maize_status_string": (ctypes.c_char_p, [_int]),
    "maize_ctx_create": (_int, [_int, ctypes.POINTER(_vp)]),
    "maize_ctx_destroy": (None, [_vp]),
    "maize_last_error": (ctypes.c_char_p, [_vp]),
    "maize_gemm_bf16": (_int, [_vp, _vp, _u32, _u32, _vp, _u32, _u32, _vp, _u32, _u32, _vp]),
    "maize_gemm_bf16_m": (_int, [_vp, _gm, _gm, _gm, _vp]),
    "maize_gemm_bf16_ld": (_int, [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _vp]),
    "maize_gemm_bf16_kn": (_int, [_vp, _vp, _u32, _u32, _vp, _u32, _u32, _vp, _u32, _u32, _vp]),
    "maize_gemm_bf16_kn_ld": (_int, [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _vp]),
    "maize_gemm_bf16_host": (_int, [_vp, _vp, _u32, _u32, _vp, _u32, _u32, _vp, _u32, _u32, _vp]),
    "maize_ctx_poll": (_int, [_vp, _vp]),
    "maize_ctx_set": (_int, [_vp, ctypes.c_char_p, _i64]),
    "maize_ctx_get": (_int, [_vp, ctypes.c_char_p, ctypes.POINTER(_i64)]),
    "maize_kernel_name": (ctypes.c_char_p, [_int]),
    "maize_pick_kernel": (_int, [_vp, _u32, _u32, _u32]),
    "maize_ctx_launch_count": (_u64, [_vp]),
    "maize_debug_wait_expires": (_int, [_vp, _u64, _vp]),
    "maize_gemm_bf16_skinny_static": (_int, [_vp, _u32, _u32, _vp, _u32, _u32, _vp, _u32, _u32, _vp, _vp,
                                             ctypes.c_char_p, ctypes.c_size_t]),
    "maize_ctx_read_profile": (_int, [_vp, ctypes.POINTER(_u64), _int, _vp]),
    "maize_mc_push": (_int, [_vp, _vp, _vp, _u64, _vp, _u32, _int, _vp]),
    "maize_mc_push_after": (_int, [_vp, _vp, _u32, _vp, _vp, _u64, _vp, _u32, _int, _vp]),
    "maize_scatter_push": (_int, [_vp, _vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _u32, _u32, _u64, _u32, _int, _vp]),
    "maize_copy_async": (_int, [_vp, _vp, _vp, _u64, _vp]),
    "maize_gemm_bf16_gated": (_int, [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _vp, _u32, _u32, _vp]),
    "maize_chain_forward": (_int, [_vp, _vp, _u32, _vp, _vp, _u64, _u64, _vp, _vp]),
    "maize_flags_wait": (_int, [_vp, _vp, _u32, _u32, _vp]),
    "maize_flag_store": (_int, [_vp, _vp, _u32, _vp]),
    "maize_mgpu_create": (_int, [_int, ctypes.POINTER(_int), ctypes.POINTER(_vp)]),
    "maize_mgpu_destroy": (None, [_vp]),
    "maize_mgpu_last_error": (ctypes.c_char_p, [_vp]),
    "maize_mgpu_size": (_int, [_vp]),
    "maize_mgpu_stream": (_vp, [_vp, _int]),
    "maize_mgpu_shard": (_int, [_vp, _u32, _int, ctypes.POINTER(_u32), ctypes.POINTER(_u32)]),
    "maize_mgpu_set": (_int, [_vp, ctypes.c_char_p, _i64]),
    "maize_gemm_bf16_nsharded": (_int, [_vp, _int, _vp, _u32, _u32, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _u32,
                                        ctypes.POINTER(_vp)]),
    "maize_gemm_bf16_nsharded_host": (_int, [_vp, _int, _vp, _u32, _u32, _vp, _u32, _vp]),
    "maize_mgpu_sync": (_int, [_vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load libmaize_gemm.so and type every entry point; raise loudly if it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m maize_b200.build` "
                "(there is no CPU fallback)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
