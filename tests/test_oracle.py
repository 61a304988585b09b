"""CPU tests of the oracle itself (no GPU): the blocked driver against a textbook loop,
against an independent float64 computation, against the committed golden vectors, and
the bf16 / RNG building blocks."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_bf16_rne_known_answers(oracle):
    L = oracle.lib()
    cases = {
        1.0: 0x3F80, -2.0: 0xC000, 0.0: 0x0000,
        1.00390625: 0x3F80,            # 1 + 2^-8: tie, rounds to even (down)
        1.01171875: 0x3F82,            # 1 + 3 * 2^-8: tie, rounds to even (up)
        1.0 + 2 ** -8 + 2 ** -20: 0x3F81,  # just above the tie
        3.3895313892515355e38: 0x7F7F,  # largest finite bf16
        float("inf"): 0x7F80,
    }
    for f, bits in cases.items():
        assert L.maize_oracle_f32_to_bf16(f) == bits, f
    assert L.maize_oracle_f32_to_bf16(3.4e38) == 0x7F80  # rounds up to inf
    nan_bits = L.maize_oracle_f32_to_bf16(float("nan"))
    assert (nan_bits & 0x7F80) == 0x7F80 and (nan_bits & 0x7F) != 0
    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32)
    ours = np.array([L.maize_oracle_f32_to_bf16(float(v)) for v in x[:2000]], dtype=np.uint16)
    assert np.array_equal(ours, oracle.f32_to_bf16(x[:2000]))


def test_fill_is_deterministic_and_sliceable(oracle):
    a = oracle.fill_bf16(7, 0, (37, 53))
    b = oracle.fill_bf16(7, 0, (37, 53))
    assert np.array_equal(a, b)
    part = oracle.fill_bf16(7, 0, (5 * 53,), first=10 * 53)
    assert np.array_equal(part, a[10:15].ravel())
    assert not np.array_equal(a, oracle.fill_bf16(8, 0, (37, 53)))
    assert not np.array_equal(a, oracle.fill_bf16(7, 1, (37, 53)))


def test_fill_distributions(oracle):
    n = oracle.bf16_to_f32(oracle.fill_bf16(0, 0, (512, 512)))
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01
    w = oracle.bf16_to_f32(oracle.fill_bf16(2, 1, (512, 512), oracle.NORMAL, 0.02))
    assert abs(w.std() - 0.02) < 3e-4
    u = oracle.bf16_to_f32(oracle.fill_bf16(1, 0, (512, 512), oracle.UNIFORM, 1.0))
    assert u.min() >= -1.0 and u.max() <= 1.0 and abs(u.mean()) < 0.01 and abs(u.std() - 3 ** -0.5) < 0.01


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 7), (16, 16, 16), (33, 47, 129), (8, 16, 2048), (70, 19, 300)])
def test_blocked_equals_textbook_loop(oracle, m, n, k):
    a = oracle.fill_bf16(11, 0, (m, k))
    b = oracle.fill_bf16(11, 1, (n, k))
    assert np.array_equal(oracle.gemm_bf16(a, b), oracle.gemm_naive(a, b))


def test_thread_count_does_not_change_bits(oracle):
    a = oracle.fill_bf16(3, 0, (64, 512))
    b = oracle.fill_bf16(3, 1, (80, 512))
    assert np.array_equal(oracle.gemm_bf16(a, b, nthreads=1), oracle.gemm_bf16(a, b, nthreads=4))


def test_against_float64(oracle):
    m, n, k = 96, 80, 1024
    a = oracle.fill_bf16(5, 0, (m, k))
    b = oracle.fill_bf16(5, 1, (n, k))
    ref64 = oracle.bf16_to_f32(a).astype(np.float64) @ oracle.bf16_to_f32(b).astype(np.float64).T
    f32 = oracle.gemm_f32out(a, b)
    assert np.max(np.abs(f32 - ref64)) < 1e-3  # fp32 running sum of ~1e3 unit-scale products
    c = oracle.bf16_to_f32(oracle.gemm_bf16(a, b))
    assert np.all(np.abs(c - ref64) <= np.abs(ref64) * 2.0 ** -8 + 1e-3)
    assert np.array_equal(oracle.gemm_bf16(a, b), oracle.f32_to_bf16(f32))


def test_empty_and_degenerate(oracle):
    z = np.zeros((0, 8), dtype=np.uint16)
    b = oracle.fill_bf16(1, 1, (4, 8))
    assert oracle.gemm_bf16(z, b).shape == (0, 4)
    a = oracle.fill_bf16(1, 0, (4, 0))
    c = oracle.gemm_bf16(a, np.zeros((3, 0), dtype=np.uint16))
    assert c.shape == (4, 3) and not c.any()  # empty sum is +0
    with pytest.raises(ValueError):
        oracle.gemm_bf16(oracle.fill_bf16(1, 0, (4, 8)), oracle.fill_bf16(1, 1, (4, 16)))


def test_check_accepts_and_rejects(oracle):
    a = oracle.fill_bf16(2, 0, (32, 256))
    b = oracle.fill_bf16(2, 1, (32, 256))
    ref = oracle.gemm_bf16(a, b)
    ma, mb = oracle.max_abs_bf16(a), oracle.max_abs_bf16(b)
    ok, err, bound, bad = oracle.check(ref, ref, 256, ma, mb)
    assert ok and err == 0 and bad == 0 and bound > 0
    broken = ref.copy()
    broken[3, 4] = 0x7FC0  # NaN
    assert not oracle.check(broken, ref, 256, ma, mb)[0]
    broken = ref.copy()
    broken[5, 6] = oracle.f32_to_bf16(np.array([1e4], dtype=np.float32))[0]
    ok, err, bound, bad = oracle.check(broken, ref, 256, ma, mb)
    assert not ok and bad == 1


def test_golden_vectors(oracle):
    """Outputs committed under tests/golden/ (made by tests/golden/make_golden.py with an independent
    numpy implementation) still come out of the oracle bit for bit."""
    index = json.loads((GOLDEN / "index.json").read_text())
    assert index["cases"]
    for case in index["cases"]:
        data = np.load(GOLDEN / case["file"])
        a = oracle.fill_bf16(case["seed"], 0, (case["m"], case["k"]), case["dist_a"], case["scale_a"])
        b = oracle.fill_bf16(case["seed"], 1, (case["n"], case["k"]), case["dist_b"], case["scale_b"])
        assert np.array_equal(a, data["a"]) and np.array_equal(b, data["b"]), case["file"]
        assert np.array_equal(oracle.gemm_bf16(a, b), data["c"]), case["file"]
