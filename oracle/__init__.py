"""CPU oracle for the BF16 GEMM path: test infrastructure, never the product.

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs
of ``bench.py`` may import this package.
"""
from .oracle import *  # noqa: F401,F403
