"""Multi-GPU parity of the N-sharded path (needs >= 2 GPUs on one box; skipped otherwise): ranks are child
processes, one per GPU, and every rank's column block of C is checked against the CPU oracle.  Several steps
with a different A each time exercise the double-buffered landing buffers and the acknowledgements."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, transport, m, n, k, steps, out_dir, extra=None):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_DEBUG="WARN")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import maize_b200
        from maize_b200.sharded import NShardedGemm
        from oracle import oracle
        ctx = maize_b200.Context(rank)
        extra = dict(extra or {})
        with_event = extra.pop("a_event", False)  # hand the step an event for "A is ready" instead of stream order
        op = NShardedGemm(m, n, k, ctx=ctx, device=dev, transport=transport, slabs=3, **extra)
        assert op.transport == transport
        b_full = oracle.fill_bf16(31, 1, (n, k))
        b_shard = torch.from_numpy(b_full[op.lo:op.hi].view(np.int16)).to(dev).view(torch.bfloat16)
        outs, keep = [], []
        for step in range(steps):
            a_root, ready = None, None
            if rank == 0:
                a = oracle.fill_bf16(100 + step, 0, (m, k))
                a_root = torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
                keep.append(a_root)  # with an event the replication may still read it after run() has returned
                if with_event:
                    ready = torch.cuda.Event()
                    ready.record()
            c = torch.full((m, op.shard_cols), float("nan"), dtype=torch.bfloat16, device=dev)
            op.run(a_root, b_shard, c, a_ready=ready)
            outs.append(c)
        dense = op.gather_c(outs[-1])  # every rank gets the whole M x N matrix of the last step
        ctx.poll()
        torch.cuda.synchronize()
        dist.barrier()
        for step, c in enumerate(outs):
            np.save(os.path.join(out_dir, f"c_{step}_{rank}.npy"), c.view(torch.int16).cpu().numpy().view(np.uint16))
        np.save(os.path.join(out_dir, f"dense_{rank}.npy"), dense.view(torch.int16).cpu().numpy().view(np.uint16))
    finally:
        dist.destroy_process_group()


def _check(oracle, tmp_path, world, m, n, k, steps, what):
    """Every step's column blocks against the oracle, and the all-gathered dense C of the last step on every rank."""
    from helpers import assert_parity
    b = oracle.fill_bf16(31, 1, (n, k))
    for step in range(steps):
        a = oracle.fill_bf16(100 + step, 0, (m, k))
        ref = oracle.gemm_bf16(a, b)
        got = np.concatenate([np.load(tmp_path / f"c_{step}_{r}.npy") for r in range(world)], axis=1)
        assert_parity(oracle, got, ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), f"{what} step {step}")
    for r in range(world):
        dense = np.load(tmp_path / f"dense_{r}.npy")
        assert dense.shape == (m, n)
        assert np.array_equal(dense, got), f"{what}: gather_c on rank {r} differs from the concatenated column blocks"


@pytest.mark.parametrize("transport", ["nccl", "multimem", "chain"])
def test_two_gpu_sharded_gemm(tmp_path, oracle, transport):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, n, k, world, steps = 1000, 1300, 520, 2, 5
    mp.spawn(_worker, args=(world, _free_port(), transport, m, n, k, steps, str(tmp_path)), nprocs=world, join=True)
    _check(oracle, tmp_path, world, m, n, k, steps, transport)


@pytest.mark.parametrize("streams", [1, 2, 4])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("a_event", [False, True])
def test_chain_variants(tmp_path, oracle, fused, streams, a_event):
    """The chain transport with small chunks: GEMMs launched per slab or (fused) as one gated launch per step,
    chunks forwarded on one stream or alternating between two, and A's readiness given by stream order or by an
    event (the replication of a step then overlaps the previous step's math; A differs from step to step here, so
    a step that read the wrong buffer would show).  Uses as many GPUs as the box has (up to 4), so that middle ranks
    (receive and forward) are covered when there are more than two."""
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    m, n, k, steps = 1500, 1300, 520, 6
    extra = dict(chain_rows=256, chain_fused=fused, chain_streams=streams, a_event=a_event)
    mp.spawn(_worker, args=(world, _free_port(), "chain", m, n, k, steps, str(tmp_path), extra), nprocs=world, join=True)
    _check(oracle, tmp_path, world, m, n, k, steps, f"chain fused={fused} streams={streams} event={a_event}")
