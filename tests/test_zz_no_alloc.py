"""The allocation-free skinny entry point, `maize_gemm_bf16_skinny_static`, called through the C ABI.

Some callers cannot allocate device memory where they need the GEMM (a service that reserves everything at
start-up, a plugin whose host owns the device memory), so this entry point keeps the kernel's scratch in a fixed
array inside the library instead of in a context.  The test runs it twice in a row, with different inputs, on a
shape that needs every slot of that array, and compares each result with what the ordinary entry point
(`maize_gemm_bf16`, scratch owned by a context) gives for the same inputs, within the tolerance of the parity
tests.  The second call finds the array as the first one left it, which is the point of calling twice.
It also checks that a shape beyond the array is refused with a message instead of being computed.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

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
            assert_parity(oracle, to_host(out), to_host(ref), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                          f"static-scratch entry, call {call}")


def test_static_scratch_entry_refuses_what_does_not_fit():
    import torch
    from maize_b200 import _ffi
    torch.cuda.set_device(0)
    lib = _ffi.load()
    too_tall = torch.zeros((33, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, too_tall, b, torch.zeros((33, 256), dtype=torch.bfloat16, device="cuda"))
    assert rc == _ffi.UNSUPPORTED and "32" in msg
    # 16 x 32768 x 4096 would need 512 partial-sum slots; the array has 256
    a = torch.zeros((16, 4096), dtype=torch.bfloat16, device="cuda")
    wide = torch.zeros((32768, 4096), dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_gemm(lib, a, wide, torch.zeros((16, 32768), dtype=torch.bfloat16, device="cuda"))
    assert rc == _ffi.UNSUPPORTED and "256" in msg and "slots" in msg
