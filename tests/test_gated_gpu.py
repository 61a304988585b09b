"""GPU tests of the gated GEMM (``maize_gemm_bf16_gated``): the loaders of the tiled kernels wait inside the
kernel for a count of landed rows of A.  On one GPU the count is preset, or raised by the HOST through pinned
memory while the kernel runs (never by another kernel on the same GPU), or never raised at all, in which case
the bounded wait must end the kernel and report a timeout."""
import threading
import time

import numpy as np
import pytest

from helpers import assert_parity, make_inputs, to_device, to_host

pytestmark = pytest.mark.gpu


def _plain_and_inputs(ctx, oracle, m, n, k, seed, force):
    import torch
    a, b = make_inputs(oracle, m, n, k, seed)
    da, db = to_device(a), to_device(b)
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", force)
    ctx.gemm(da, db, out=want)
    ctx.poll()
    return a, b, da, db, want


@pytest.mark.parametrize("force", [0, 1, 2, 3, 4, 5, 10, 12])
@pytest.mark.parametrize("m,n,k,rows", [(300, 520, 264, 128), (1500, 1300, 520, 256), (2048, 4096, 512, 1024)])
def test_preset_count_is_bit_identical(ctx, oracle, m, n, k, rows, force):
    """With every chunk already counted the gated call is the plain call, on each tiled kernel; the count may
    also be ahead (a later step's value) and the base may sit near the 32-bit wrap."""
    import torch
    try:
        a, b, da, db, want = _plain_and_inputs(ctx, oracle, m, n, k, 41, force)
        for base, ahead in ((0, 0), (7, 3), (0xFFFFFFFE, 0)):
            count = np.array([(base + -(-m // rows) + ahead) & 0xFFFFFFFF], dtype=np.uint32)
            word = torch.from_numpy(count.view(np.int32)).cuda()
            got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            ctx.gemm_gated(da, db, got, word.data_ptr(), base, rows)
            ctx.poll()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, n, k, rows, force, base)
    finally:
        ctx.set("force_kernel", 0)
    ref = oracle.gemm_bf16(a, b)
    assert_parity(oracle, to_host(want), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), "gated, preset")


@pytest.mark.parametrize("force", [0, 1, 5, 10, 12])
def test_host_raises_the_count_while_the_kernel_runs(ctx, oracle, force):
    """Nothing has landed at launch; the host counts the chunks in mapped pinned memory, a few at a time, and the
    kernel's loaders follow.  The result is bit-identical to the plain call."""
    import torch
    m, n, k, rows = 4096, 2048, 1024, 256
    chunks = m // rows
    base = 1000
    word = torch.full((1,), base, dtype=torch.int32).pin_memory()
    view = word.numpy()
    try:
        a, b, da, db, want = _plain_and_inputs(ctx, oracle, m, n, k, 42, force)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()

        def deliver():
            for c in range(1, chunks + 1):
                time.sleep(0.0005)
                view[0] = base + c

        t = threading.Thread(target=deliver)
        ctx.gemm_gated(da, db, got, word.data_ptr(), base, rows)
        t.start()
        t.join()
        ctx.poll()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    finally:
        ctx.set("force_kernel", 0)


@pytest.mark.parametrize("force", [1, 5, 12])
def test_count_that_never_comes_times_out(ctx, oracle, force):
    """Half of A is counted and the rest never is: the kernel ends by itself after the budget, the status says
    timeout, and the next call on the same context is correct."""
    import torch
    import maize_b200
    m, n, k, rows = 2048, 1024, 256, 256
    budget = ctx.get("timeout_ns")
    try:
        a, b, da, db, want = _plain_and_inputs(ctx, oracle, m, n, k, 43, force)
        word = torch.tensor([4], dtype=torch.int32, device="cuda")  # 4 of 8 chunks
        got = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ctx.set("timeout_ns", 3_000_000)  # 3 ms
        ctx.gemm_gated(da, db, got, word.data_ptr(), 0, rows)
        with pytest.raises(maize_b200.MaizeError) as e:
            ctx.poll()
        assert e.value.status == maize_b200._ffi.TIMEOUT
        ctx.set("timeout_ns", budget)
        ctx.poll()  # the status word was cleared
        # rows whose chunks were counted may have been computed; the context works as before
        again = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ctx.gemm(da, db, out=again)
        ctx.poll()
        assert torch.equal(again.view(torch.int16), want.view(torch.int16))
    finally:
        ctx.set("force_kernel", 0)
        ctx.set("timeout_ns", budget)


def test_gated_rejects_bad_arguments(ctx):
    import torch
    import maize_b200
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((256, 256), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    word = torch.zeros(2, dtype=torch.int32, device="cuda")
    for ptr, rows in ((0, 128), (word.data_ptr() + 2, 128), (word.data_ptr(), 0)):
        with pytest.raises(maize_b200.MaizeError) as e:
            ctx.gemm_gated(a, b, c, ptr, 0, rows)
        assert e.value.status == maize_b200._ffi.INVALID_ARG
