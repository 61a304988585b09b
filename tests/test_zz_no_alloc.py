"""The allocation-free skinny entry point, `maize_gemm_bf16_skinny_static`, called through the C ABI.

Some callers cannot allocate device memory where they need the GEMM (a service that reserves everything at
start-up, a plugin whose host owns the device memory), so this entry point keeps the kernel's scratch in a fixed
array inside the library instead of in a context.  The test runs it twice in a row, with different inputs, on a
shape that needs every slot of that array, and compares each result with what the ordinary entry point
(`maize_gemm_bf16`, scratch owned by a context) gives for the same inputs AND with the CPU oracle, within the
tolerance of the parity tests.  The second call finds the array as the first one left it, which is the point of
calling twice.  Further cases: no status buffer (the status word then lives in the array), a second device when
the box has one, free device memory unchanged by a call, K = 0, and shapes beyond the array, which are refused
with a message instead of being computed.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes
import re

import numpy as np
import pytest

from helpers import assert_parity, make_inputs, to_device, to_host

pytestmark = pytest.mark.gpu


def _static_gemm(lib, da, db, dc, status=None):
    import torch
    err = ctypes.create_string_buffer(256)
    m, k = da.shape
    n = db.shape[0]
    rc = lib.maize_gemm_bf16_skinny_static(da.data_ptr(), m, k, db.data_ptr(), n, k, dc.data_ptr(), m, n,
                                           torch.cuda.current_stream().cuda_stream,
                                           status.data_ptr() if status is not None else None, err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("m,n,k", [(16, 16384, 4096), (7, 1000, 520)])
def test_static_scratch_entry_matches_context_entry_twice(oracle, m, n, k):
    import torch
    import maize_b200
    from maize_b200 import _ffi
    torch.cuda.set_device(0)
    lib = _ffi.load()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    with maize_b200.Context(0) as ctx:
        for call, seed in enumerate((41, 42)):
            a, b = make_inputs(oracle, m, n, k, seed, scale_b=0.05)
            da, db = to_device(a), to_device(b)
            ref = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            ctx.gemm_raw(da.data_ptr(), m, k, db.data_ptr(), n, k, ref.data_ptr(), m, n)  # existing entry point
            ctx.poll()
            out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            rc, msg = _static_gemm(lib, da, db, out, status)
            assert rc == _ffi.OK, msg
            torch.cuda.synchronize()
            assert int(status[0]) == 0, f"device status {status.tolist()} on call {call}"
            ma, mb = oracle.max_abs_bf16(a), oracle.max_abs_bf16(b)
            assert_parity(oracle, to_host(out), to_host(ref), k, ma, mb, f"static-scratch entry vs context entry, call {call}")
            assert_parity(oracle, to_host(out), oracle.gemm_bf16(a, b), k, ma, mb, f"static-scratch entry vs oracle, call {call}")


def test_static_scratch_entry_without_status_buffer_and_without_allocating(oracle):
    """device_status = NULL: the kernel's status word is the one inside the library's array.  Free device memory
    is the same before and after each call once every tensor of the test exists (the first call on a device may
    still load the library's GPU code, which is why it is made before the measurement)."""
    import torch
    from maize_b200 import _ffi
    torch.cuda.set_device(0)
    lib = _ffi.load()
    m, n, k = 16, 16384, 4096
    cases = []
    for seed in (43, 44, 45):
        a, b = make_inputs(oracle, m, n, k, seed, scale_b=0.05)
        cases.append((a, b, to_device(a), to_device(b), torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")))
    rc, msg = _static_gemm(lib, cases[0][2], cases[0][3], cases[0][4])  # warm-up: module load, address look-up
    assert rc == _ffi.OK, msg
    torch.cuda.synchronize()
    for a, b, da, db, out in cases[1:]:
        free_before, _ = torch.cuda.mem_get_info()
        rc, msg = _static_gemm(lib, da, db, out)
        assert rc == _ffi.OK, msg
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across a call"
    for a, b, da, db, out in cases:
        assert_parity(oracle, to_host(out), oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                      "static-scratch entry, no status buffer")


def test_static_scratch_entry_on_a_second_device(oracle):
    """Every device has its own copy of the array and its own address for it: a call made with device 1 current
    must use device 1's."""
    import torch
    from maize_b200 import _ffi
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = _ffi.load()
    m, n, k = 16, 4096, 1024
    a, b = make_inputs(oracle, m, n, k, 46, scale_b=0.05)
    ref = oracle.gemm_bf16(a, b)
    try:
        for dev in (1, 0, 1):
            torch.cuda.set_device(dev)
            da, db = to_device(a).to(f"cuda:{dev}"), to_device(b).to(f"cuda:{dev}")
            out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=f"cuda:{dev}")
            status = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
            rc, msg = _static_gemm(lib, da, db, out, status)
            assert rc == _ffi.OK, msg
            torch.cuda.synchronize(dev)
            assert int(status[0]) == 0
            assert_parity(oracle, to_host(out), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), f"device {dev}")
    finally:
        torch.cuda.set_device(0)


def test_static_scratch_entry_k_zero_gives_zero():
    import torch
    from maize_b200 import _ffi
    torch.cuda.set_device(0)
    lib = _ffi.load()
    a = torch.zeros((5, 0), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((9, 0), dtype=torch.bfloat16, device="cuda")
    c = torch.full((5, 9), 3.0, dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, a, b, c)
    assert rc == _ffi.OK, msg
    torch.cuda.synchronize()
    assert not to_host(c).any()


def test_static_scratch_entry_refuses_what_does_not_fit():
    import torch
    from maize_b200 import _ffi
    torch.cuda.set_device(0)
    lib = _ffi.load()
    too_tall = torch.zeros((33, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, too_tall, b, torch.zeros((33, 256), dtype=torch.bfloat16, device="cuda"))
    assert rc == _ffi.UNSUPPORTED and "32" in msg

    def needs(msg):
        got = re.search(r"needs (\d+) partial-sum slots and (\d+) counters; the static scratch holds (\d+) and (\d+)", msg)
        assert got, msg
        return tuple(int(x) for x in got.groups())

    # 16 x 32768 x 4096 on 148 SMs: 128 tiles of 3 parts = 384 partial-sum slots (the array has 256), 512 counters
    a = torch.zeros((16, 4096), dtype=torch.bfloat16, device="cuda")
    wide = torch.zeros((32768, 4096), dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, a, wide, torch.zeros((16, 32768), dtype=torch.bfloat16, device="cuda"))
    assert rc == _ffi.UNSUPPORTED
    slots, counters, have_slots, have_counters = needs(msg)
    assert slots > have_slots == 256 and counters <= have_counters
    del wide
    # N beyond 65536 with a short K: whole tiles per CTA (no slots needed), but more counters than the array has
    a = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    long_n = torch.zeros((65792, 64), dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, a, long_n, torch.zeros((8, 65792), dtype=torch.bfloat16, device="cuda"))
    assert rc == _ffi.UNSUPPORTED
    slots, counters, have_slots, have_counters = needs(msg)
    assert counters > have_counters == 1024 and slots <= have_slots
