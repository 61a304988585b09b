"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Ordered from the safest launch to the largest."""
import numpy as np
import pytest

from helpers import CONFIGS, assert_parity, make_inputs, to_device, to_host

pytestmark = pytest.mark.gpu


def run_case(ctx, oracle, m, n, k, seed=0, force=0, **dist):
    import torch
    a, b = make_inputs(oracle, m, n, k, seed, **dist)
    da, db = to_device(a), to_device(b)
    dc = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", force)
    try:
        ctx.gemm_raw(da.data_ptr(), m, k, db.data_ptr(), n, k, dc.data_ptr(), m, n)
        ctx.poll()
    finally:
        ctx.set("force_kernel", 0)
    ref = oracle.gemm_bf16(a, b)
    return assert_parity(oracle, to_host(dc), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                         what=f"{m}x{n}x{k} kernel {force}")


def test_bounded_wait_returns_timeout(ctx):
    """A wait that nothing satisfies ends by itself and is reported, and the context stays usable."""
    import maize_b200
    ctx.debug_wait_expires(200_000)  # 0.2 ms budget
    with pytest.raises(maize_b200.MaizeError) as e:
        ctx.poll()
    assert e.value.status == maize_b200._ffi.TIMEOUT
    ctx.poll()  # the status word was cleared


def test_settings_read_back(ctx):
    """Every key of maize_ctx_set can be read with maize_ctx_get (no kernel is launched here)."""
    for key, value in (("group_rows", 1024), ("b_static", 1), ("push_threads", 256), ("max_ctas", 100),
                       ("force_kernel", 2), ("debug_flags", 0), ("chain_streams", 3), ("repack_bytes", 4096), ("pdl", 0),
                       ("serpentine", 0), ("tail_split", 0), ("tma_store", 0), ("tma_promotion", 2)):
        before = ctx.get(key)
        try:
            ctx.set(key, value)
            assert ctx.get(key) == value, key
        finally:
            ctx.set(key, before)
    assert ctx.get("sm_count") > 0 and ctx.get("device") == 0 and ctx.get("profile") == 0


def test_debug_flags_need_profile(ctx):
    """The diagnostic switches make results wrong on purpose: they are refused unless profiling is on."""
    import maize_b200
    with pytest.raises(maize_b200.MaizeError) as e:
        ctx.set("debug_flags", 1)
    assert e.value.status == maize_b200._ffi.INVALID_ARG
    ctx.set("profile", 1)
    try:
        ctx.set("debug_flags", 1)
        assert ctx.get("debug_flags") == 1
    finally:
        ctx.set("profile", 0)
    assert ctx.get("debug_flags") == 0  # turning profiling off clears them


def test_stream_k_recovers_after_a_timeout(ctx, oracle):
    """A stream-K launch whose waits run out may leave arrival counters half-way (one part of a tile published,
    another given up).  maize_ctx_poll re-zeroes them when it reports the timeout, so the next launch on the same
    context is right.  Three CTAs share two tiles of 1024 k-blocks; the budgets below lie around the time one CTA
    needs for a third and for two thirds of a tile, so that some pieces finish and others give up."""
    import torch
    import maize_b200
    m, n, k = 16, 512, 65536
    a, b = make_inputs(oracle, m, n, k, 33, scale_b=0.05)
    da, db = to_device(a), to_device(b)
    ref = oracle.gemm_bf16(a, b)
    timed_out = 0
    for budget_ns in (20_000, 60_000, 120_000, 250_000):
        ctx.set("force_kernel", 7)
        ctx.set("max_ctas", 3)
        ctx.set("timeout_ns", budget_ns)
        try:
            junk = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            ctx.gemm(da, db, out=junk)
            try:
                ctx.poll()
            except maize_b200.MaizeError as e:
                assert e.status == maize_b200._ffi.TIMEOUT
                timed_out += 1
        finally:
            ctx.set("timeout_ns", 2_000_000_000)
        try:
            out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            ctx.gemm(da, db, out=out)
            ctx.poll()
        finally:
            ctx.set("max_ctas", 0)
            ctx.set("force_kernel", 0)
        assert_parity(oracle, to_host(out), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                      f"after a launch with a {budget_ns} ns budget")
    assert timed_out >= 1, "no budget was short enough to make a wait run out"


@pytest.mark.parametrize("force", [1, 2, 3, 4, 5, 6])
def test_single_tile_single_kblock(ctx, oracle, force):
    run_case(ctx, oracle, 128, 256, 64, seed=10, force=force)


@pytest.mark.parametrize("force", [1, 2, 3, 4, 5, 6])
def test_ring_wraps(ctx, oracle, force):
    # more k-blocks than stages: every barrier changes phase several times
    run_case(ctx, oracle, 128, 256, 64 * 21, seed=11, force=force)


@pytest.mark.parametrize("force", [1, 2, 3, 4, 5, 6])
def test_many_tiles_per_cta(ctx, oracle, force):
    # more tiles than SMs for every variant: both TMEM accumulator buffers and their phases cycle
    run_case(ctx, oracle, 128 * 10, 256 * 9, 256, seed=12, force=force)


@pytest.mark.parametrize("m,n,k", [
    (1, 1, 8), (1, 8, 8), (7, 5, 16), (130, 250, 72), (127, 33, 520), (300, 1000, 136), (129, 257, 64),
    (128, 255, 128), (513, 77, 1032), (64, 4096, 256), (2000, 24, 512),
])
@pytest.mark.parametrize("force", [0, 1, 2, 3, 4, 5, 6])
def test_ragged_edges(ctx, oracle, m, n, k, force):
    run_case(ctx, oracle, m, n, k, seed=13, force=force)


@pytest.mark.parametrize("m,n,k", [
    (1, 128, 64), (16, 128, 64), (16, 128, 640), (16, 4096, 1024), (13, 1000, 520), (3, 77, 72), (16, 16384, 256),
    (32, 2048, 512), (20, 2050, 520), (64, 1024, 1024), (50, 999, 264), (128, 4096, 512), (100, 300, 136),
    (16, 300000, 64), (8, 128 * 300, 4096),
])
def test_skinny_shapes(ctx, oracle, m, n, k):
    """M <= 128 goes to the stream-K kernels: whole tiles, split tiles (2 and more parts), ragged N and K,
    more tiles than SMs, and the whole-tile fallback for very many tiles."""
    assert "skinny" in ctx.pick_kernel(m, n, k)
    run_case(ctx, oracle, m, n, k, seed=19)
    run_case(ctx, oracle, m, n, k, seed=20)  # again: the arrival counters were reset by the first launch


@pytest.mark.parametrize("force,m", [(7, 16), (7, 32), (7, 5), (8, 16), (8, 33), (8, 128), (8, 100)])
def test_skinny_variants_forced(ctx, oracle, force, m):
    run_case(ctx, oracle, m, 256 * 37, 64 * 29, seed=21, force=force)
    run_case(ctx, oracle, m, 333, 200, seed=22, force=force)
    run_case(ctx, oracle, m, 256 * 75, 4104, seed=24, force=force)  # 65 k-blocks, split tiles
    run_case(ctx, oracle, m, 1001, 136, seed=25, force=force)  # odd N: 2-byte aligned C rows


@pytest.mark.parametrize("m,n,k", [
    (16, 16384, 4096), (1, 9472, 64), (32, 4096, 4096), (7, 1000, 520), (16, 18944, 1088), (20, 33, 72),
    (16, 8191, 136), (32, 16385, 264),
])
def test_skinny_pair_split(ctx, oracle, m, n, k):
    """K split over a CTA pair with the halves added through shared memory: odd and single k-block counts,
    every tile width from 32 to 256, ragged last tiles, unaligned C rows."""
    run_case(ctx, oracle, m, n, k, seed=27, force=9)
    run_case(ctx, oracle, m, n, k, seed=28, force=9)


@pytest.mark.parametrize("m,n,k", [
    (128, 16384, 4096), (33, 9472, 64), (100, 4096, 4096), (64, 1000, 520), (77, 18944, 1088), (40, 33, 72),
    (128, 8191, 136), (96, 16385, 264), (16, 4096, 1024),
])
def test_skinny_pair_split_tall(ctx, oracle, m, n, k):
    """The pair-split decode kernel for 32 < M <= 128 (A tile loaded once, halves exchanged through the leader's
    whole ring): odd and single k-block counts, tile widths from 32 to 256, ragged last tiles, unaligned C rows,
    and an M <= 32 shape forced through it."""
    run_case(ctx, oracle, m, n, k, seed=37, force=11)
    run_case(ctx, oracle, m, n, k, seed=38, force=11)


def test_skinny_pair_tall_is_chosen_and_deterministic(ctx, oracle):
    import torch
    m, n, k = 100, 4096, 4096
    assert "skinny_pair_m128" in ctx.pick_kernel(m, n, k)
    run_case(ctx, oracle, m, n, k, seed=39)
    a, b = make_inputs(oracle, m, n, k, 40)
    da, db = to_device(a), to_device(b)
    outs = [ctx.gemm(da, db).clone() for _ in range(3)]
    ctx.poll()
    assert all(torch.equal(outs[0].view(torch.int16), o.view(torch.int16)) for o in outs[1:])


def test_skinny_pair_with_dependent_launch(ctx, oracle):
    """Back-to-back decode launches with programmatic dependent launch: A of launch i+1 is produced by a kernel
    that runs between the GEMMs, so the dependency wait is what keeps the result right; B is declared static."""
    import torch
    m, n, k = 16, 16384, 1024
    a, b = make_inputs(oracle, m, n, k, 30, scale_b=0.05)
    da, db = to_device(a), to_device(b)
    ref1 = oracle.gemm_bf16(a, b)
    a2 = oracle.f32_to_bf16(oracle.bf16_to_f32(a) * 2.0)
    ref2 = oracle.gemm_bf16(a2, b)
    ctx.set("pdl", 1)
    ctx.set("b_static", 1)
    try:
        outs = []
        x = da.clone()
        for i in range(6):
            c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            ctx.gemm(x, db, out=c)
            outs.append(c)
            x = da * 2 if i % 2 == 0 else da.clone()  # the next launch's A comes from a kernel in between
        ctx.poll()
    finally:
        ctx.set("pdl", 1)  # the library's default
        ctx.set("b_static", 0)
    for i, c in enumerate(outs):
        ref = ref1 if i % 2 == 0 else ref2
        assert_parity(oracle, to_host(c), ref, k, 2 * oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), f"launch {i}")


@pytest.mark.parametrize("pdl", [1, 0])
@pytest.mark.parametrize("force", [0, 1, 6, 10])
def test_tiled_kernels_with_dependent_launch(ctx, oracle, force, pdl):
    """"pdl" on the tiled kernels: each launch may start its set-up while the previous kernel drains, and must
    still see that kernel's output.  A chain of GEMMs where C of one launch is A of the next (several times, back
    to back, nothing in between) is the case that goes wrong if the dependency wait is missing or misplaced."""
    import torch
    m, n, k = 1536, 1024, 1024  # C is m x n, and n == k, so C can be the next A
    a, b = make_inputs(oracle, m, n, k, 34, scale_b=1.0 / 32)
    da, db = to_device(a), to_device(b)
    ctx.set("pdl", pdl)  # 1 is the default; 0 = ordinary launches
    ctx.set("force_kernel", force)
    try:
        xs = [da]
        for _ in range(4):
            xs.append(ctx.gemm(xs[-1], db))
        ctx.poll()
    finally:
        ctx.set("pdl", 1)  # the library's default
        ctx.set("force_kernel", 0)
    for i in range(4):
        x = to_host(xs[i])
        assert_parity(oracle, to_host(xs[i + 1]), oracle.gemm_bf16(x, b), k, oracle.max_abs_bf16(x), oracle.max_abs_bf16(b),
                      f"link {i} of the chain, kernel {force}")


def test_skinny_pair_rejects_more_than_one_wave(ctx):
    import torch
    import maize_b200
    a = torch.zeros((16, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((74 * 256 + 1, 64), dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", 9)
    try:
        with pytest.raises(maize_b200.MaizeError) as e:
            ctx.gemm(a, b)
        assert e.value.status == maize_b200._ffi.UNSUPPORTED
    finally:
        ctx.set("force_kernel", 0)


def test_skinny_is_deterministic(ctx, oracle):
    import torch
    a, b = make_inputs(oracle, 16, 16384, 4096, 23)
    da, db = to_device(a), to_device(b)
    outs = [ctx.gemm(da, db).clone() for _ in range(3)]
    ctx.poll()
    assert all(torch.equal(outs[0].view(torch.int16), o.view(torch.int16)) for o in outs[1:])


def test_forced_skinny_rejects_tall_a(ctx):
    import torch
    import maize_b200
    a = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", 7)
    try:
        with pytest.raises(maize_b200.MaizeError) as e:
            ctx.gemm(a, b)
        assert e.value.status == maize_b200._ffi.UNSUPPORTED
    finally:
        ctx.set("force_kernel", 0)


@pytest.mark.parametrize("force", [0, 1, 2, 3, 5, 6])
@pytest.mark.parametrize("m,n,k", [
    (128, 256, 64), (128, 256, 64 * 9), (256, 512, 256), (300, 1000, 136), (513, 264, 1032), (7, 8, 16),
    (130, 248, 72), (1280, 2304, 256), (2000, 24, 512), (64, 4096, 100),
])
def test_b_stored_k_by_n(ctx, oracle, m, n, k, force):
    """B given K x N row-major (the reference demo's layout): loaded as 64-column boxes, MN-major MMA operand.
    N must be a multiple of 8 (row pitch); K is free."""
    import torch
    a = oracle.fill_bf16(29, 0, (m, k))
    b_nk = oracle.fill_bf16(29, 1, (n, k))
    ref = oracle.gemm_bf16(a, b_nk)
    da = to_device(a)
    db_kn = to_device(np.ascontiguousarray(b_nk.T))  # K x N
    lda_pad = (k + 7) // 8 * 8
    if lda_pad != k:  # A's row pitch must be a multiple of 8 elements: embed A in a padded buffer
        buf = torch.zeros((m, lda_pad), dtype=torch.bfloat16, device="cuda")
        buf[:, :k] = da
        da = buf[:, :k]
    dc = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", force)
    try:
        ctx.gemm_kn(da, db_kn, out=dc)
        ctx.poll()
    finally:
        ctx.set("force_kernel", 0)
    assert_parity(oracle, to_host(dc), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b_nk),
                  f"K x N B, {m}x{n}x{k}, kernel {force}")


@pytest.mark.parametrize("force,m", [(9, 16), (9, 32), (9, 1), (11, 128), (11, 33), (11, 16), (0, 16), (0, 100)])
@pytest.mark.parametrize("n,k", [(16384, 4096), (4096, 1024), (1000, 520), (9472, 64), (8200, 264)])
def test_decode_shapes_with_b_stored_k_by_n(ctx, oracle, force, m, n, k):
    """The pair-split decode kernels with B given K x N: tiles widened to a multiple of 64 columns, loaded as
    64-column boxes, MN-major MMA operand; ragged N and K, single and odd k-block counts."""
    import torch
    a = oracle.fill_bf16(44, 0, (m, k))
    b_nk = oracle.fill_bf16(44, 1, (n, k), scale=0.05)
    ref = oracle.gemm_bf16(a, b_nk)
    da = to_device(a)
    db_kn = to_device(np.ascontiguousarray(b_nk.T))  # K x N
    dc = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    if force == 0:
        assert "skinny_pair" in ctx.pick_kernel(m, n, k)
    ctx.set("force_kernel", force)
    try:
        ctx.gemm_kn(da, db_kn, out=dc)
        ctx.poll()
    finally:
        ctx.set("force_kernel", 0)
    assert_parity(oracle, to_host(dc), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b_nk),
                  f"decode, K x N B, {m}x{n}x{k}, kernel {force}")


def test_b_k_by_n_full_config(ctx, oracle):
    """Config c1 (4096^3, the reference demo's own size) with B in the demo's K x N layout."""
    m = n = k = 4096
    a = oracle.fill_bf16(0, 0, (m, k))
    b_nk = oracle.fill_bf16(0, 1, (n, k))
    dc = ctx.gemm_kn(to_device(a), to_device(np.ascontiguousarray(b_nk.T)))
    ctx.poll()
    assert_parity(oracle, to_host(dc), oracle.gemm_bf16(a, b_nk), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b_nk))


def test_canaries_around_c(ctx, oracle):
    """Nothing is written outside C: rows of padding between C rows (ldc > N) and guard bands stay intact."""
    import torch
    m, n, k, ldc = 200, 333, 136, 340
    a, b = make_inputs(oracle, m, n, k, 14)
    da, db = to_device(a), to_device(b)
    guard = 1024
    buf = torch.full((guard + m * ldc + guard,), 7.0, dtype=torch.bfloat16, device="cuda")
    c_ptr = buf.data_ptr() + guard * 2
    ctx.gemm_ld(da.data_ptr(), k, db.data_ptr(), k, c_ptr, ldc, m, n, k)
    ctx.poll()
    host = to_host(buf)
    seven = to_host(torch.full((1,), 7.0, dtype=torch.bfloat16))[0]
    assert np.all(host[:guard] == seven) and np.all(host[guard + m * ldc:] == seven)
    body = host[guard:guard + m * ldc].reshape(m, ldc)
    assert np.all(body[:, n:] == seven)
    assert_parity(oracle, np.ascontiguousarray(body[:, :n]), oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a),
                  oracle.max_abs_bf16(b), "strided C")


@pytest.mark.parametrize("force", [1, 2, 3, 5, 6, 10])
@pytest.mark.parametrize("tma_store", [1, 0])
def test_canaries_around_c_with_aligned_rows(ctx, oracle, force, tma_store):
    """C rows 16-byte aligned (ldc % 8 == 0) but narrower than the pitch and with ragged M and N: the tiled kernels
    write such a C through shared memory and TMA stores, which must clip at M and N exactly; the direct-store
    path ("tma_store" = 0) is held to the same."""
    import torch
    m, n, k, ldc = 300, 328, 200, 336
    a, b = make_inputs(oracle, m, n, k, 41)
    da, db = to_device(a), to_device(b)
    guard = 1024
    buf = torch.full((guard + m * ldc + guard,), 7.0, dtype=torch.bfloat16, device="cuda")
    c_ptr = buf.data_ptr() + guard * 2
    ctx.set("force_kernel", force)
    ctx.set("tma_store", tma_store)
    try:
        ctx.gemm_ld(da.data_ptr(), k, db.data_ptr(), k, c_ptr, ldc, m, n, k)
        ctx.poll()
    finally:
        ctx.set("force_kernel", 0)
        ctx.set("tma_store", 1)
    host = to_host(buf)
    seven = to_host(torch.full((1,), 7.0, dtype=torch.bfloat16))[0]
    assert np.all(host[:guard] == seven) and np.all(host[guard + m * ldc:] == seven)
    body = host[guard:guard + m * ldc].reshape(m, ldc)
    assert np.all(body[:, n:] == seven)
    assert_parity(oracle, np.ascontiguousarray(body[:, :n]), oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a),
                  oracle.max_abs_bf16(b), f"aligned strided C, kernel {force}, tma_store {tma_store}")


def test_strided_operands(ctx, oracle):
    """Row slabs / column slices as used by the N-sharded path: lda, ldb > K and ldc > N."""
    import torch
    m, n, k = 260, 300, 192
    a, b = make_inputs(oracle, m, n, 2 * k, 15)
    da, db = to_device(a), to_device(b)
    full_c = torch.zeros((m, 2 * n), dtype=torch.bfloat16, device="cuda")
    out = ctx.gemm(da[:, k:], db[:, :k], out=full_c[:, n:])
    ctx.poll()
    assert out.data_ptr() == full_c[:, n:].data_ptr()
    ref = oracle.gemm_bf16(np.ascontiguousarray(a[:, k:]), np.ascontiguousarray(b[:, :k]))
    assert_parity(oracle, to_host(full_c[:, n:]), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), "strided")
    assert not to_host(full_c[:, :n]).any()


def test_k_zero_and_empty(ctx, oracle):
    import torch
    c = torch.full((5, 9), 3.0, dtype=torch.bfloat16, device="cuda")
    a = torch.zeros((5, 0), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((9, 0), dtype=torch.bfloat16, device="cuda")
    ctx.gemm(a, b, out=c)
    ctx.poll()
    assert not to_host(c).any()
    ctx.gemm_raw(0, 0, 64, 0, 9, 64, 0, 0, 9)  # M == 0: nothing to do, no pointer is touched


def test_argument_errors(ctx):
    import torch
    import maize_b200
    E = maize_b200._ffi
    a = torch.zeros((16, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((16, 8), dtype=torch.bfloat16, device="cuda")
    cases = [
        (lambda: ctx.gemm_raw(a.data_ptr(), 16, 64, b.data_ptr(), 8, 32, c.data_ptr(), 16, 8), E.INVALID_ARG),
        (lambda: ctx.gemm_raw(a.data_ptr(), 16, 64, b.data_ptr(), 8, 64, c.data_ptr(), 16, 9), E.INVALID_ARG),
        (lambda: ctx.gemm_raw(a.data_ptr(), 16, 64, b.data_ptr(), 8, 64, 0, 16, 8), E.INVALID_ARG),
        (lambda: ctx.gemm_raw(0, 16, 64, b.data_ptr(), 8, 64, c.data_ptr(), 16, 8), E.INVALID_ARG),
        (lambda: ctx.gemm_raw(a.data_ptr(), 16, 60, b.data_ptr(), 8, 60, c.data_ptr(), 16, 8), E.UNSUPPORTED),
        (lambda: ctx.gemm_raw(a.data_ptr() + 2, 15, 64, b.data_ptr(), 8, 64, c.data_ptr(), 15, 8), E.UNSUPPORTED),
        (lambda: ctx.gemm_ld(a.data_ptr(), 32, b.data_ptr(), 64, c.data_ptr(), 8, 16, 8, 64), E.INVALID_ARG),
        (lambda: ctx.gemm_ld(a.data_ptr(), 64, b.data_ptr(), 64, c.data_ptr(), 4, 16, 8, 64), E.INVALID_ARG),
    ]
    for call, status in cases:
        with pytest.raises(maize_b200.MaizeError) as e:
            call()
        assert e.value.status == status
    ctx.poll()


def test_matrix_bundle_entry_point(ctx, oracle):
    import torch
    import maize_b200
    m, n, k = 96, 72, 128
    a, b = make_inputs(oracle, m, n, k, 16)
    da, db = to_device(a), to_device(b)
    dc = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    M = maize_b200.Matrix
    ctx.gemm_matrices(M.from_tensor(da), M.from_tensor(db), M.new(dc.data_ptr(), m, n))
    ctx.poll()
    assert_parity(oracle, to_host(dc), oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b))


def test_host_entry_point(ctx, oracle):
    """Host buffers in and out through maize_gemm_bf16_host (pinned and pageable)."""
    import torch
    m, n, k = 300, 520, 264
    a, b = make_inputs(oracle, m, n, k, 17)
    ref = oracle.gemm_bf16(a, b)
    c = np.zeros((m, n), dtype=np.uint16)
    ctx.gemm_host(a.ctypes.data, m, k, b.ctypes.data, n, k, c.ctypes.data, m, n)
    ctx.poll()
    assert_parity(oracle, c, ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), "pageable host")
    pa = torch.from_numpy(a.view(np.int16)).pin_memory()
    pb = torch.from_numpy(b.view(np.int16)).pin_memory()
    pc = torch.zeros((m, n), dtype=torch.int16).pin_memory()
    ctx.gemm_host(pa.data_ptr(), m, k, pb.data_ptr(), n, k, pc.data_ptr(), m, n)
    ctx.poll()
    assert np.array_equal(pc.numpy().view(np.uint16), c)


def test_host_entry_point_pipelined(ctx, oracle):
    """Large enough for the slab pipeline (B first, A in row slabs, C rows read back as they finish), ragged M."""
    import torch
    m, n, k = 5000, 3000, 2048
    a, b = make_inputs(oracle, m, n, k, 26)
    ref = oracle.gemm_bf16(a, b)
    pa = torch.from_numpy(a.view(np.int16)).pin_memory()
    pb = torch.from_numpy(b.view(np.int16)).pin_memory()
    pc = torch.zeros((m, n), dtype=torch.int16).pin_memory()
    for _ in range(2):  # twice: staging and events are reused
        pc.zero_()
        ctx.gemm_host(pa.data_ptr(), m, k, pb.data_ptr(), n, k, pc.data_ptr(), m, n)
        ctx.poll()
        assert_parity(oracle, pc.numpy().view(np.uint16), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b),
                      "pipelined host entry")


@pytest.mark.parametrize("m,n,k", [(300, 520, 264), (5000, 3000, 2048)])
def test_host_entry_point_keeps_a_static_b_on_the_device(ctx, oracle, m, n, k):
    """With "b_static" a second call with the same host B re-uses the copy on the device (A changes, B does not
    cross PCIe again); once the promise is withdrawn a changed B is uploaded again.  Both the single-copy and the
    pipelined form."""
    import torch
    a1, b = make_inputs(oracle, m, n, k, 35)
    a2 = oracle.fill_bf16(36, 0, (m, k))
    pa = torch.from_numpy(a1.view(np.int16).copy()).pin_memory()
    pb = torch.from_numpy(b.view(np.int16).copy()).pin_memory()
    pc = torch.zeros((m, n), dtype=torch.int16).pin_memory()
    ma, mb = max(oracle.max_abs_bf16(a1), oracle.max_abs_bf16(a2)), oracle.max_abs_bf16(b)
    ctx.set("b_static", 1)
    try:
        for a in (a1, a2, a1):
            pa.copy_(torch.from_numpy(a.view(np.int16)))
            pc.zero_()
            ctx.gemm_host(pa.data_ptr(), m, k, pb.data_ptr(), n, k, pc.data_ptr(), m, n)
            ctx.poll()
            assert_parity(oracle, pc.numpy().view(np.uint16), oracle.gemm_bf16(a, b), k, ma, mb, "static B")
    finally:
        ctx.set("b_static", 0)
    b2 = oracle.fill_bf16(37, 1, (n, k))
    pb.copy_(torch.from_numpy(b2.view(np.int16)))
    ctx.gemm_host(pa.data_ptr(), m, k, pb.data_ptr(), n, k, pc.data_ptr(), m, n)
    ctx.poll()
    assert_parity(oracle, pc.numpy().view(np.uint16), oracle.gemm_bf16(a1, b2), k, ma, oracle.max_abs_bf16(b2), "new B")


@pytest.mark.parametrize("force", [0, 1, 6])
@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_baseline_configs_full(ctx, oracle, name, force):
    m, n, k, da, sa, db, sb, seed = CONFIGS[name]
    run_case(ctx, oracle, m, n, k, seed=seed, force=force, dist_a=da, scale_a=sa, dist_b=db, scale_b=sb)


def test_deterministic_across_launches(ctx, oracle):
    import torch
    m, n, k = 1024, 2048, 512
    a, b = make_inputs(oracle, m, n, k, 18)
    da, db = to_device(a), to_device(b)
    c1 = ctx.gemm(da, db)
    c2 = ctx.gemm(da, db)
    ctx.poll()
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))


@pytest.mark.parametrize("name", ["c4", "c5", "t"])
def test_large_configs_sampled_and_properties(ctx, oracle, name):
    """Full-size shapes: sampled rows against the oracle, the whole matrix against an fp32 matmul on the
    GPU (a library call used as a second checker only), and linearity in A as a size-independent property."""
    import torch
    m, n, k, da_, sa, db_, sb, seed = CONFIGS[name]
    a, b = make_inputs(oracle, m, n, k, seed, da_, sa, db_, sb)
    da, db = to_device(a), to_device(b)
    dc = ctx.gemm(da, db)
    ctx.poll()
    ma, mb = oracle.max_abs_bf16(a), oracle.max_abs_bf16(b)
    rows = np.unique(np.concatenate([np.arange(0, 8), np.arange(m - 8, m),
                                     np.random.default_rng(seed).integers(0, m, 48)]))
    ref_rows = oracle.gemm_bf16(np.ascontiguousarray(a[rows]), b)
    got_rows = to_host(dc[torch.from_numpy(rows).cuda()])
    assert_parity(oracle, got_rows, ref_rows, k, ma, mb, f"{name} sampled rows")
    # whole matrix against fp32 matmul of the widened operands, in row slabs to bound memory
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        bf = db.float()
        tol = 1e-4 * float(np.sqrt(k)) * ma * mb
        for r0 in range(0, m, 2048):
            ref = da[r0:r0 + 2048].float() @ bf.T
            err = (dc[r0:r0 + 2048].float() - ref).abs() - ref.abs() * 2.0 ** -7
            assert float(err.max()) <= tol, f"{name} rows {r0}..: {float(err.max())} > {tol}"
        del bf
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    # linearity: (2A) B^T == 2 (A B^T) exactly (power-of-two scaling commutes with every rounding)
    c2 = ctx.gemm(da * 2, db)
    ctx.poll()
    assert torch.equal((dc * 2).view(torch.int16), c2.view(torch.int16))
