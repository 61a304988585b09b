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
        op = NShardedGemm(m, n, k, ctx=ctx, device=dev, transport=transport, slabs=3, **(extra or {}))
        assert op.transport == transport
        b_full = oracle.fill_bf16(31, 1, (n, k))
        b_shard = torch.from_numpy(b_full[op.lo:op.hi].view(np.int16)).to(dev).view(torch.bfloat16)
        outs = []
        for step in range(steps):
            a_root = None
            if rank == 0:
                a = oracle.fill_bf16(100 + step, 0, (m, k))
                a_root = torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
            c = torch.full((m, op.shard_cols), float("nan"), dtype=torch.bfloat16, device=dev)
            op.run(a_root, b_shard, c)
            outs.append(c)
        ctx.poll()
        torch.cuda.synchronize()
        dist.barrier()
        for step, c in enumerate(outs):
            np.save(os.path.join(out_dir, f"c_{step}_{rank}.npy"), c.view(torch.int16).cpu().numpy().view(np.uint16))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["nccl", "multimem", "chain"])
def test_two_gpu_sharded_gemm(tmp_path, oracle, transport):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import assert_parity
    m, n, k, world, steps = 1000, 1300, 520, 2, 5
    mp.spawn(_worker, args=(world, _free_port(), transport, m, n, k, steps, str(tmp_path)), nprocs=world, join=True)
    b = oracle.fill_bf16(31, 1, (n, k))
    for step in range(steps):
        a = oracle.fill_bf16(100 + step, 0, (m, k))
        ref = oracle.gemm_bf16(a, b)
        got = np.concatenate([np.load(tmp_path / f"c_{step}_{r}.npy") for r in range(world)], axis=1)
        assert_parity(oracle, got, ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), f"{transport} step {step}")


@pytest.mark.parametrize("streams", [1, 2])
@pytest.mark.parametrize("fused", [False, True])
def test_chain_enqueued_by_the_library(tmp_path, oracle, fused, streams):
    """The chain transport with the whole step's forwarding enqueued by one library call and small chunks, with the
    GEMMs launched per slab or (fused) as one gated launch per step; uses as many GPUs as the box has (up to 4), so
    that middle ranks (receive and forward) are covered when there are > 2."""
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    from helpers import assert_parity
    m, n, k, steps = 1500, 1300, 520, 5
    extra = dict(chain_rows=256, chain_in_library=True, chain_fused=fused, chain_streams=streams)
    mp.spawn(_worker, args=(world, _free_port(), "chain", m, n, k, steps, str(tmp_path), extra), nprocs=world, join=True)
    b = oracle.fill_bf16(31, 1, (n, k))
    for step in range(steps):
        a = oracle.fill_bf16(100 + step, 0, (m, k))
        ref = oracle.gemm_bf16(a, b)
        got = np.concatenate([np.load(tmp_path / f"c_{step}_{r}.npy") for r in range(world)], axis=1)
        assert_parity(oracle, got, ref, k, oracle.max_abs_bf16(a), oracle.max_abs_bf16(b), f"chain in library, step {step}")
