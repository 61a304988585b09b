"""The single-process multi-GPU entry points of the C ABI (maize_mgpu_*): argument checks that need no GPU, and on
a box with >= 2 GPUs the N-sharded GEMM on device buffers and on host buffers against the CPU oracle, over several
steps with a different A each (the landing buffers are reused from step to step), with either end of the device
list as the root."""
import ctypes

import numpy as np
import pytest

from helpers import assert_parity


def test_create_refuses_bad_arguments_or_reports_no_device():
    from maize_b200 import _ffi
    lib = _ffi.load()
    h = ctypes.c_void_p()
    assert lib.maize_mgpu_create(0, (ctypes.c_int * 1)(0), ctypes.byref(h)) == _ffi.INVALID_ARG
    assert lib.maize_mgpu_create(2, None, ctypes.byref(h)) == _ffi.INVALID_ARG
    assert lib.maize_mgpu_create(1, (ctypes.c_int * 1)(0), None) == _ffi.INVALID_ARG
    assert lib.maize_mgpu_sync(None) == _ffi.INVALID_ARG
    assert lib.maize_mgpu_size(None) == 0
    st = lib.maize_mgpu_create(2, (ctypes.c_int * 2)(0, 0), ctypes.byref(h))  # the same device twice
    assert st in (_ffi.INVALID_ARG, _ffi.NO_DEVICE)
    import torch
    if not torch.cuda.is_available():
        assert lib.maize_mgpu_create(1, (ctypes.c_int * 1)(0), ctypes.byref(h)) == _ffi.NO_DEVICE


def _dev_tensor(u16, dev):
    import torch
    return torch.from_numpy(u16.view(np.int16)).to(f"cuda:{dev}").view(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("root_last", [False, True])
@pytest.mark.parametrize("overlap", [False, True])
def test_nsharded_on_device_buffers(oracle, root_last, overlap):
    import torch
    from maize_b200.mgpu import MultiGpu
    G = min(torch.cuda.device_count(), 4)
    if G < 2:
        pytest.skip("needs two GPUs")
    m, n, k, steps = 1500, 1300, 520, 5
    root = G - 1 if root_last else 0
    b = oracle.fill_bf16(31, 1, (n, k))
    with MultiGpu(list(range(G))) as mg:
        assert len(mg) == G
        mg.set("chunk_rows", 256)
        mg.set("chain_streams", 2)
        if overlap:
            mg.set("a_on_stream", 0)  # every A below is complete before its call: forwarding may run ahead
        bounds = [mg.shard(n, g) for g in range(G)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n and all(bounds[g][1] == bounds[g + 1][0] for g in range(G - 1))
        a_host = [oracle.fill_bf16(100 + s, 0, (m, k)) for s in range(steps)]
        a_dev = [_dev_tensor(a, root) for a in a_host]
        a_local = [None if g == root else torch.empty((m, k), dtype=torch.bfloat16, device=f"cuda:{g}") for g in range(G)]
        b_sh = [_dev_tensor(np.ascontiguousarray(b[lo:hi]), g) for g, (lo, hi) in enumerate(bounds)]
        c_sh = [[torch.full((m, hi - lo), float("nan"), dtype=torch.bfloat16, device=f"cuda:{g}")
                 for g, (lo, hi) in enumerate(bounds)] for _ in range(steps)]
        for g in range(G):
            torch.cuda.synchronize(g)
        for s in range(steps):
            mg.gemm_nsharded(root, a_dev[s], a_local, b_sh, c_sh[s], n)
        mg.sync()
        for s in range(steps):
            got = np.concatenate([c.view(torch.int16).cpu().numpy().view(np.uint16) for c in c_sh[s]], axis=1)
            assert_parity(oracle, got, oracle.gemm_bf16(a_host[s], b), k, oracle.max_abs_bf16(a_host[s]),
                          oracle.max_abs_bf16(b), f"step {s}, root {root}, overlap {overlap}")


@pytest.mark.gpu
def test_nsharded_on_host_buffers(oracle):
    import torch
    from maize_b200.mgpu import MultiGpu
    G = min(torch.cuda.device_count(), 4)
    if G < 2:
        pytest.skip("needs two GPUs")
    with MultiGpu(list(range(G))) as mg:
        for (m, n, k), seed in (((1100, 1301, 520), 7), ((300, 77, 264), 8), ((2100, 2050, 1032), 9)):
            a = oracle.fill_bf16(seed, 0, (m, k))
            b = oracle.fill_bf16(seed, 1, (n, k))
            c = np.full((m, n), 0xFFFF, dtype=np.uint16)
            mg.gemm_nsharded_host(0, a.ctypes.data, m, k, b.ctypes.data, n, c.ctypes.data)
            assert_parity(oracle, c, oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                          f"host buffers {m}x{n}x{k}")


@pytest.mark.gpu
def test_single_device_handle(oracle):
    """n = 1 degenerates to one plain GEMM on that device."""
    from maize_b200.mgpu import MultiGpu
    m, n, k = 300, 520, 264
    a = oracle.fill_bf16(3, 0, (m, k))
    b = oracle.fill_bf16(3, 1, (n, k))
    c = np.zeros((m, n), dtype=np.uint16)
    with MultiGpu([0]) as mg:
        mg.gemm_nsharded_host(0, a.ctypes.data, m, k, b.ctypes.data, n, c.ctypes.data)
    assert_parity(oracle, c, oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b))
