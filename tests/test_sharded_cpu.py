"""Host logic of the N-sharded path on CPU ranks (gloo, world size 2): the partition of B / C, the
row slabs of A, and the slab-by-slab broadcast.  The multiply itself is injected (the CPU oracle), since
the CUDA kernels need a GPU; what is under test here is everything around them."""
import os
import socket

import numpy as np
import pytest

from maize_b200.sharded import plan_slabs, shard_bounds, slab_bounds


def test_shard_bounds_cover_and_balance():
    for n in (1, 7, 3967, 16384, 28672):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard_bounds(16384, 8, 3) == (6144, 8192)
    assert shard_bounds(28672, 8, 7) == (25088, 28672)
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_slab_bounds():
    assert slab_bounds(16384, 8) == [(i * 2048, (i + 1) * 2048) for i in range(8)]
    s = slab_bounds(4111, 8)
    assert s[0][0] == 0 and s[-1][1] == 4111 and all(a[1] == b[0] for a, b in zip(s, s[1:]))
    assert all((hi - lo) % 128 == 0 for lo, hi in s[:-1]) and len(s) <= 8
    assert slab_bounds(16, 8) == [(0, 16)]
    assert slab_bounds(0, 4) == []


def test_plan_slabs_covers_and_aligns():
    for m, cols, k in [(16384, 2048, 16384), (16384, 8192, 16384), (8192, 3584, 8192), (8192, 14336, 8192),
                       (4111, 1984, 4104), (100, 64, 64)]:
        plan = plan_slabs(m, cols, k)
        assert plan[0][0] == 0 and plan[-1][1] == m
        assert all(a[1] == b[0] for a, b in zip(plan, plan[1:]))
        assert all(lo % 256 == 0 for lo, _ in plan) and 1 <= len(plan) <= 16
    # 8 GPUs on 16384^3: 8 column tiles per shard, 74 tile pairs in flight.  Every slab but the ones at
    # the two ends should fill its waves almost completely.
    plan = plan_slabs(16384, 2048, 16384)
    fills = []
    for lo, hi in plan:
        tiles = (hi - lo) // 256 * 8
        fills.append(tiles / (-(-tiles // 74) * 74))
    assert sum(f * (hi - lo) for f, (lo, hi) in zip(fills, plan)) / 16384 > 0.9
    # the model prefers several slabs when the transfer is comparable to the compute, one when it is free
    assert len(plan) >= 3
    assert len(plan_slabs(16384, 2048, 16384, bcast_gbs=1e9)) <= 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, out_dir):
    import torch
    import torch.distributed as dist
    from oracle import oracle
    from maize_b200.sharded import NShardedGemm

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def as_u16(t):
            return t.contiguous().view(torch.int16).numpy().view(np.uint16)

        def cpu_gemm(a, b, c):
            c.copy_(torch.from_numpy(oracle.gemm_bf16(as_u16(a), as_u16(b)).view(np.int16)).view(torch.bfloat16))

        a_full = oracle.fill_bf16(21, 0, (m, k))
        b_full = oracle.fill_bf16(21, 1, (n, k))
        op = NShardedGemm(m, n, k, slabs=3, gemm_fn=cpu_gemm)
        a_root = torch.from_numpy(a_full.view(np.int16)).view(torch.bfloat16) if rank == 0 else None
        b_shard = torch.from_numpy(b_full[op.lo:op.hi].view(np.int16)).view(torch.bfloat16)
        c_shard = torch.zeros((m, op.shard_cols), dtype=torch.bfloat16)
        for _ in range(2):  # twice: the landing buffer is reused
            op.run(a_root, b_shard, c_shard)
        np.save(os.path.join(out_dir, f"c{rank}.npy"), as_u16(c_shard))
        dense = op.gather_c(c_shard)
        assert dense.shape == (m, n)
        np.save(os.path.join(out_dir, f"dense{rank}.npy"), as_u16(dense))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_gemm_matches_unsharded(tmp_path, oracle):
    import torch.multiprocessing as mp
    m, n, k, world = 300, 143, 96, 2
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    ref = oracle.gemm_bf16(oracle.fill_bf16(21, 0, (m, k)), oracle.fill_bf16(21, 1, (n, k)))
    got = np.concatenate([np.load(tmp_path / f"c{r}.npy") for r in range(world)], axis=1)
    assert np.array_equal(got, ref)
    for r in range(world):  # the all-gathered dense C is the same on every rank (uneven shards: 72 + 71 columns)
        assert np.array_equal(np.load(tmp_path / f"dense{r}.npy"), ref)
