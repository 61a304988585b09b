"""N-sharded multi-GPU GEMM: one process per GPU, A broadcast over NCCL, C stays sharded.

The reference has no multi-GPU code; its only decomposition is the grid-stride of column
panels of B over ``ctaid.y`` (crates/maize_tile/src/gmem/col_panel.rs:88-124,
group/by_block.rs:51-75).  The same split is lifted one level up: rank ``r`` of ``G`` owns
rows ``[r*N/G, (r+1)*N/G)`` of B (N x K, K-major, so a contiguous block) and produces the
matching column block of C into its own dense M x (N/G) buffer.  Output columns are
independent, so the only exchange is the replication of A: no reduction.

A is cut into row slabs.  The broadcasts of all slabs are queued first (NCCL runs them in
order on its own stream); the GEMM of slab i only waits for broadcast i, so the transfer of
slab i+1 overlaps the math of slab i and only the first slab's transfer is exposed.  The
broadcast lands in this GPU's own memory; kernels only ever read local memory.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows of B / columns of C owned by ``rank``: near-equal contiguous blocks, larger ones first."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def slab_bounds(m: int, slabs: int, align: int = 128) -> List[Tuple[int, int]]:
    """Cut M rows into at most ``slabs`` row slabs whose sizes are multiples of ``align`` (the
    kernel's tile height) except the last, so that no slab adds a ragged tile row of its own."""
    if m <= 0:
        return []
    slabs = max(1, slabs)
    rows = -(-m // slabs)
    rows = -(-rows // align) * align
    out = []
    lo = 0
    while lo < m:
        hi = min(m, lo + rows)
        out.append((lo, hi))
        lo = hi
    return out


class NShardedGemm:
    """``C[:, shard] = A @ B[shard].T`` on every rank, A living on ``root`` before the call.

    ``gemm_fn(a_slab, b_shard, c_slab)`` defaults to the CUDA GEMM of this package; tests on
    CPU ranks (gloo) pass their own to exercise the partition and the exchange.
    """

    def __init__(self, m: int, n: int, k: int, group=None, root: int = 0, slabs: int = 8,
                 gemm_fn: Optional[Callable] = None, device=None, ctx=None):
        import torch
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.root = root
        self.m, self.n, self.k = m, n, k
        self.lo, self.hi = shard_bounds(n, self.world, self.rank)
        self.slabs = slab_bounds(m, slabs if self.world > 1 else 1)
        self.device = device
        if gemm_fn is None:
            from .gemm import default_context
            self.ctx = ctx or default_context(torch.device(device).index if device is not None else None)
            gemm_fn = lambda a, b, c: self.ctx.gemm(a, b, out=c)  # noqa: E731
        self.gemm_fn = gemm_fn
        self._a_local = None

    @property
    def shard_cols(self) -> int:
        return self.hi - self.lo

    def a_buffer(self, like):
        """This rank's landing buffer for A (the root uses its own A in place)."""
        import torch
        if self._a_local is None:
            self._a_local = torch.empty((self.m, self.k), dtype=like.dtype, device=like.device)
        return self._a_local

    def run(self, a_root, b_shard, c_shard):
        """One step: replicate A from the root slab by slab and multiply as slabs arrive.

        ``a_root`` is the M x K matrix on the root and ignored elsewhere (may be None);
        ``b_shard`` is this rank's (hi-lo) x K block of B; ``c_shard`` is M x (hi-lo).
        """
        if self.world == 1:
            self.gemm_fn(a_root, b_shard, c_shard)
            return c_shard
        is_root = self.rank == self.root
        a = a_root if is_root else self.a_buffer(b_shard)
        src = self.dist.get_global_rank(self.group, self.root) if self.group is not None else self.root
        works = []
        for lo, hi in self.slabs:
            works.append(self.dist.broadcast(a[lo:hi], src=src, group=self.group, async_op=True))
        for (lo, hi), work in zip(self.slabs, works):
            if not is_root:
                work.wait()  # the compute stream waits for this slab only
            self.gemm_fn(a[lo:hi], b_shard, c_shard[lo:hi])
        if is_root:
            for work in works:
                work.wait()  # A must not be overwritten before the sends have read it
        return c_shard
