"""maize_b200: a B200-native BF16 GEMM behind maize's GEMM call shape.

``gemm(a, b)`` computes ``a @ b.T`` (A is M x K, B is N x K, both bf16, fp32
accumulation, bf16 result) with hand-written sm_100a kernels reached through the C
ABI of ``include/maize_gemm.h``.  There is no CPU path: importing works anywhere,
computing needs the built library and a B200.
"""
from . import tile  # noqa: F401
from ._ffi import LIB_PATH, STATUS_NAMES  # noqa: F401
from .gemm import Context, MaizeError, Matrix, default_context, gemm, gemm_skinny_static  # noqa: F401

__all__ = ["Context", "MaizeError", "Matrix", "default_context", "gemm", "gemm_skinny_static", "tile", "LIB_PATH"]
