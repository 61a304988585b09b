"""Shared pieces of the parity tests: seeded inputs, tensor <-> raw-bf16 views, the two bounds."""
from __future__ import annotations

import math

import numpy as np

# BASELINE configs: (M, N, K, dist_a, scale_a, dist_b, scale_b, seed)
NORMAL, UNIFORM = 0, 1
CONFIGS = {
    "c1": (4096, 4096, 4096, NORMAL, 1.0, NORMAL, 1.0, 0),
    "c2": (4111, 3967, 4104, UNIFORM, 1.0, UNIFORM, 1.0, 1),
    "c3": (16, 16384, 4096, NORMAL, 1.0, NORMAL, 0.02, 2),
    "c4": (16384, 16384, 16384, NORMAL, 1.0, NORMAL, 1.0, 3),
    "c5": (8192, 28672, 8192, NORMAL, 1.0, NORMAL, 0.02, 4),
    "t": (8192, 8192, 8192, NORMAL, 1.0, NORMAL, 1.0, 5),
}


def make_inputs(oracle, m, n, k, seed=0, dist_a=NORMAL, scale_a=1.0, dist_b=NORMAL, scale_b=1.0):
    a = oracle.fill_bf16(seed, 0, (m, k), dist_a, scale_a)
    b = oracle.fill_bf16(seed, 1, (n, k), dist_b, scale_b)
    return a, b


def to_device(u16: np.ndarray):
    """numpy uint16 (raw bf16 bits) -> torch bfloat16 CUDA tensor with the same bits."""
    import torch
    return torch.from_numpy(u16.view(np.int16)).cuda().view(torch.bfloat16)


def to_host(t) -> np.ndarray:
    """torch bfloat16 tensor -> numpy uint16 raw bits."""
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def assert_parity(oracle, c_gpu: np.ndarray, c_ref: np.ndarray, k: int, max_a: float, max_b: float, what=""):
    """Two checks against the oracle.

    (1) The path's stated tolerance: |C - C_ref| <= 1e-2 * sqrt(K) * max|a| * max|b| + one bf16 ulp of C_ref.
    (2) A much tighter bug-catching bound.  Both sides accumulate in fp32 and differ only in summation
        order, so they may disagree by the final rounding (one bf16 ulp, 2^-7 relative) plus fp32
        reassociation noise; 1e-4 * sqrt(K) * max|a| * max|b| is far above that noise yet far below the
        effect of one dropped or duplicated 16-wide k-step (about 4 * typical |a| * |b|).
    """
    ok, err, bound, bad = oracle.check(c_gpu, c_ref, k, max_a, max_b)
    assert ok, f"{what}: {bad} elements beyond the path tolerance; max |err| {err:.4g} vs bound {bound:.4g}"
    g = oracle.bf16_to_f32(c_gpu).astype(np.float64)
    r = oracle.bf16_to_f32(c_ref).astype(np.float64)
    tight = np.abs(r) * 2.0 ** -7 + 1e-4 * math.sqrt(max(k, 1)) * max_a * max_b
    diff = np.abs(g - r)
    worst = int(np.argmax(diff - tight))
    assert np.all(diff <= tight), (
        f"{what}: tight bound violated at flat index {worst}: gpu {g.flat[worst]} ref {r.flat[worst]} "
        f"({int(np.sum(diff > tight))} elements)")
    return err, bound
