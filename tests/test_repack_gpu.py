"""GPU tests of the pitch-aligning pre-pass: operands whose row pitch is not a multiple of 128 bytes are copied to
an aligned pitch (into scratch the context holds, "repack_bytes") ahead of a GEMM that is long enough for the copy
to pay; the result must not change by a bit."""
import numpy as np
import pytest

from helpers import assert_parity, make_inputs, to_device, to_host

pytestmark = pytest.mark.gpu

DEFAULT_SCRATCH = 128 << 20


@pytest.mark.parametrize("m,n,k", [(1100, 1300, 520), (2055, 1983, 2056), (4111, 3967, 4104), (4096, 4096, 4096)])
def test_repack_is_bit_identical(ctx, oracle, m, n, k):
    import torch
    a, b = make_inputs(oracle, m, n, k, 61)
    da, db = to_device(a), to_device(b)
    plain = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert ctx.get("repack_bytes") == DEFAULT_SCRATCH  # a context holds this much by default
    ctx.set("repack_bytes", 0)
    try:
        ctx.gemm(da, db, out=plain)
        ctx.poll()
    finally:
        ctx.set("repack_bytes", DEFAULT_SCRATCH)
    launches = ctx.launch_count
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.gemm(da, db, out=got)
    ctx.poll()
    used = ctx.launch_count - launches
    assert torch.equal(got.view(torch.int16), plain.view(torch.int16))
    # one copy launch (A and B together) and the GEMM when the pitch is misaligned and the problem is large enough,
    # else the GEMM alone
    assert used == (2 if (m, n, k) == (4111, 3967, 4104) else 1), used
    ref = oracle.gemm_bf16(a, b)
    assert_parity(oracle, to_host(got), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), "repacked")


def test_repack_with_two_different_unaligned_pitches_and_static_b(ctx, oracle):
    """lda != ldb, both not multiples of 128 bytes (A and B are column slices of wider buffers); with "b_static" the
    copy of B is made once and reused while A changes from call to call."""
    import torch
    m, n, k = 4000, 3900, 4104
    a, b = make_inputs(oracle, m, n, k, 62)
    wa = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")   # pitch 8224 B
    wb = torch.zeros((n, k + 24), dtype=torch.bfloat16, device="cuda")  # pitch 8256 B
    wa[:, :k] = to_device(a)
    wb[:, :k] = to_device(b)
    ref = oracle.gemm_bf16(a, b)
    a2 = oracle.f32_to_bf16(oracle.bf16_to_f32(a) * 0.5)
    ref2 = oracle.gemm_bf16(a2, b)
    ctx.set("b_static", 1)
    try:
        launches = ctx.launch_count
        c1 = ctx.gemm(wa[:, :k], wb[:, :k])
        wa[:, :k] = to_device(a2)
        c2 = ctx.gemm(wa[:, :k], wb[:, :k])
        ctx.poll()
        assert ctx.launch_count - launches == 4  # (copy of A and B, GEMM), (copy of A only, GEMM)
    finally:
        ctx.set("b_static", 0)
    ma, mb = oracle.max_abs_bf16(a), oracle.max_abs_bf16(b)
    assert_parity(oracle, to_host(c1), ref, k, ma, mb, "first call")
    assert_parity(oracle, to_host(c2), ref2, k, ma, mb, "second call, B's copy reused")
    # without the promise B is copied again: same bits
    c3 = ctx.gemm(wa[:, :k], wb[:, :k])
    ctx.poll()
    assert np.array_equal(to_host(c3), to_host(c2))
