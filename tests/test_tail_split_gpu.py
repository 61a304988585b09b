"""GPU parity tests of the CTA-pair kernel whose last, partial round of tiles is split along K (kernel id 10,
forced: the selection never picks it yet)."""
import pytest

from test_gemm_gpu import run_case

pytestmark = pytest.mark.gpu

TAIL = 10


@pytest.mark.parametrize("m,n,k", [
    (2304, 2304, 2048),   # 81 tiles on 74 pairs: one full round, 7 tiles split in 2
    (2304, 2304, 4096),   # the same, split in 4
    (512, 1024, 8192),    # 8 tiles, fewer than pairs: every tile split in 8
    (300, 520, 2056),     # ragged single-round problem: 6 tiles split in 2, K not a multiple of 128
    (2304, 2304, 512),    # K too short to split: the last round is an ordinary round
    (4736, 4096, 1024),   # 19 x 16 = 304 tiles = 4 full rounds and 8 tiles... split 8 needs 64 steps: stays 1
])
def test_tail_split_parity(ctx, oracle, m, n, k):
    run_case(ctx, oracle, m, n, k, seed=51, force=TAIL)


def test_tail_split_twice_is_bit_identical(ctx, oracle):
    """The counters return to zero and the parts are added in part order whoever arrives last."""
    import torch
    from helpers import make_inputs, to_device
    m, n, k = 2304, 2304, 4096
    a, b = make_inputs(oracle, m, n, k, 52)
    da, db = to_device(a), to_device(b)
    outs = []
    ctx.set("force_kernel", TAIL)
    try:
        for _ in range(3):
            c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            ctx.gemm(da, db, out=c)
            ctx.poll()
            outs.append(c)
    finally:
        ctx.set("force_kernel", 0)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))
