"""A plain-C program (tests/c_abi/harness.c: C11, no CUDA headers, no Python) linked against libmaize_gemm.so:
the drop-in boundary as a compiled-language caller sees it.  The CPU tests check that it compiles with
-pedantic, links every symbol it uses, answers the host-only calls and refuses loudly without a device; the
GPU test runs parity cases through maize_gemm_bf16_host against the oracle."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    from maize_b200 import _ffi
    from oracle import oracle
    lib = Path(_ffi.LIB_PATH)
    if not lib.exists():
        pytest.fail(f"{lib} is missing: build it with `python -m maize_b200.build`")
    oracle.build()
    oracle_dir = ROOT / "oracle" / "_build"
    exe = tmp_path_factory.mktemp("c_abi") / "harness"
    cmd = ["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-O2", "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "c_abi" / "harness.c"), "-o", str(exe), "-L", str(lib.parent), "-lmaize_gemm",
           "-L", str(oracle_dir), "-loracle", f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{oracle_dir}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def _run(exe, *args):
    env = dict(os.environ, OMP_NUM_THREADS=str(min(16, os.cpu_count() or 1)))
    return subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True, timeout=600, env=env)


def test_host_only_calls(harness):
    r = _run(harness, "--selftest")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failure(s)" in r.stdout


def test_no_device_is_reported_not_computed(harness):
    """Without a GPU the library has nothing to fall back on: the program says so and exits 77."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    r = _run(harness, 300, 520, 264)
    assert r.returncode == 77, r.stdout + r.stderr
    assert "no CUDA device" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(300, 520, 264), (16, 4096, 1024), (1100, 1300, 520), (4096, 4096, 2048)])
def test_parity_through_the_c_program(harness, m, n, k):
    """Single-copy path, decode shape, ragged shape, and a problem large enough for the pipelined copies."""
    r = _run(harness, m, n, k, 7)
    assert r.returncode == 0, r.stdout + r.stderr
    assert " 0 violation(s)" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1100, 1300, 520), (2500, 2050, 1032)])
def test_multi_gpu_parity_through_the_c_program(harness, m, n, k):
    """maize_gemm_bf16_nsharded_host from plain C on every GPU of the box (up to 4; one GPU degenerates to a plain
    GEMM), two calls with a different A."""
    import torch
    g = max(1, min(torch.cuda.device_count(), 4))
    r = _run(harness, "--mgpu", g, m, n, k, 11)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count(" 0 violation(s)") == 2 and f"{g} device(s)" in r.stdout
