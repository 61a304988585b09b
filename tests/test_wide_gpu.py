"""GPU parity tests of the CTA-pair kernel with a 256 x 512 tile (kernel id 12: one accumulator filling tensor
memory, two MMAs per k-step sharing the A operand, the next tile started on the half of the accumulator that the
epilogue has already drained)."""
import numpy as np
import pytest

from helpers import assert_parity, make_inputs, to_device, to_host
from test_gemm_gpu import run_case

pytestmark = pytest.mark.gpu

WIDE = 12


@pytest.mark.parametrize("m,n,k", [
    (256, 512, 64),        # one tile, one k-block: the head of the tile is the whole tile
    (256, 512, 192),       # fewer k-blocks than ring stages
    (256, 512, 64 * 21),   # the ring wraps several times
    (256 * 5, 512 * 40, 256),   # 200 tiles on 74 pairs: the accumulator halves change hands many times
    (300, 1000, 136),      # ragged M, N and K; C rows 16-byte aligned: TMA stores clip
    (513, 1031, 1032),     # odd N: the direct-store epilogue
    (130, 250, 72), (1, 8, 8), (2000, 24, 512), (129, 513, 64),
    (2304, 4096, 2048),    # several full rounds
])
def test_wide_tile_parity(ctx, oracle, m, n, k):
    run_case(ctx, oracle, m, n, k, seed=71, force=WIDE)


def test_wide_tile_is_bit_identical_to_the_pair_kernel(ctx, oracle):
    """Same MMA shape and the same ascending-k order per element: the 256 x 512 kernel must give the very bits the
    256 x 256 pair kernel gives."""
    import torch
    m, n, k = 1536, 3072, 4096
    a, b = make_inputs(oracle, m, n, k, 72)
    da, db = to_device(a), to_device(b)
    outs = {}
    for force in (6, WIDE):
        ctx.set("force_kernel", force)
        try:
            outs[force] = ctx.gemm(da, db)
            ctx.poll()
        finally:
            ctx.set("force_kernel", 0)
    assert torch.equal(outs[6].view(torch.int16), outs[WIDE].view(torch.int16))


def test_wide_tile_is_chosen_when_enabled(ctx, oracle):
    """With "wide_tile" on (the default), long-K shapes whose rounds of 256 x 512 tiles are nearly full take the wide
    kernel; others stay with the 256 x 256 pair kernel."""
    assert ctx.get("wide_tile") in (0, 1)
    before = ctx.get("wide_tile")
    ctx.set("wide_tile", 1)
    try:
        assert ctx.pick_kernel(8192, 8192, 8192) == "sm100_2cta_256x512x64_s4"
        assert ctx.pick_kernel(16384, 16384, 16384) == "sm100_2cta_256x512x64_s4"
        ctx.set("wide_max_gflop", 2200)
        try:
            assert ctx.pick_kernel(16384, 16384, 16384) == "sm100_2cta_256x256x128_s3"  # capped by the caller
        finally:
            ctx.set("wide_max_gflop", 1000000)
        assert ctx.pick_kernel(4096, 4096, 4096) == "sm100_2cta_256x512x64_s4"    # 128 wide tiles: two rounds, 86 % full
        assert ctx.pick_kernel(8192, 3584, 8192) == "sm100_2cta_256x256x128_s3"   # 224 wide tiles: four rounds, 76 % full
        assert ctx.pick_kernel(8192, 8192, 512) == "sm100_2cta_256x256x128_s3"    # K too short
        m, n, k = 2048, 4608, 2048  # 8 x 9 = 72 tiles: one round of 74 pairs, nearly full
        assert ctx.pick_kernel(m, n, k) == "sm100_2cta_256x512x64_s4"
        run_case(ctx, oracle, m, n, k, seed=73)
    finally:
        ctx.set("wide_tile", before)


def test_wide_tile_canaries(ctx, oracle):
    import torch
    m, n, k, ldc = 300, 840, 200, 848
    a, b = make_inputs(oracle, m, n, k, 74)
    da, db = to_device(a), to_device(b)
    guard = 1024
    buf = torch.full((guard + m * ldc + guard,), 7.0, dtype=torch.bfloat16, device="cuda")
    ctx.set("force_kernel", WIDE)
    try:
        ctx.gemm_ld(da.data_ptr(), k, db.data_ptr(), k, buf.data_ptr() + guard * 2, ldc, m, n, k)
        ctx.poll()
    finally:
        ctx.set("force_kernel", 0)
    host = to_host(buf)
    seven = to_host(torch.full((1,), 7.0, dtype=torch.bfloat16))[0]
    assert np.all(host[:guard] == seven) and np.all(host[guard + m * ldc:] == seven)
    body = host[guard:guard + m * ldc].reshape(m, ldc)
    assert np.all(body[:, n:] == seven)
    assert_parity(oracle, np.ascontiguousarray(body[:, :n]), oracle.gemm_bf16(a, b), k, oracle.max_abs_bf16(a),
                  oracle.max_abs_bf16(b), "wide tile, strided C")


def test_wide_tile_needs_rows_of_c_that_tma_can_store(ctx, oracle):
    """The wide tile's epilogue is exposed, so the heuristic takes it only when C leaves through TMA stores: the
    same shape with an odd row pitch of C runs on the 256 x 256 pair kernel ("last_kernel" tells which ran)."""
    import torch
    m, n, k = 2048, 4608, 2048
    a = oracle.fill_bf16(75, 0, (m, k))
    b = oracle.fill_bf16(75, 1, (n, k))
    ref = oracle.gemm_bf16(a, b)
    da, db = to_device(a), to_device(b)
    dense = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.gemm(da, db, out=dense)
    assert ctx.last_kernel == "sm100_2cta_256x512x64_s4"
    wide = torch.full((m, n + 3), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.gemm(da, db, out=wide[:, :n])
    assert ctx.last_kernel == "sm100_2cta_256x256x128_s3"
    ctx.poll()
    assert torch.equal(dense.view(torch.int16), wide[:, :n].view(torch.int16))
    assert torch.isnan(wide[:, n:]).all()
    assert_parity(oracle, to_host(dense), ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), "wide tile, dense C")
