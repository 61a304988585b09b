"""N-sharded multi-GPU GEMM: one process per GPU, A replicated over NVLink, C stays sharded.

The reference has no multi-GPU code; its only decomposition is the grid-stride of column
panels of B over ``ctaid.y`` (crates/maize_tile/src/gmem/col_panel.rs:88-124,
group/by_block.rs:51-75).  The same split is lifted one level up: rank ``r`` of ``G`` owns
rows ``[r*N/G, (r+1)*N/G)`` of B (N x K, K-major, so a contiguous block) and produces the
matching column block of C into its own dense M x (N/G) buffer.  Output columns are
independent, so the only exchange is the replication of A: no reduction.

A is cut into row slabs; the GEMM of slab i only waits for slab i to land, so the transfer of
slab i+1 overlaps the math of slab i.  Three transports ("auto" = ``chain`` where symmetric memory can be set
up, else ``nccl``):

* ``multimem`` (needs an NVSwitch multicast mapping): the root pushes each
  slab ONCE through the switch with ``multimem.st`` into symmetric landing buffers on every GPU
  and publishes a slab counter the same way (``mc_stages=1``, the default); receivers run no
  copy kernel, only a one-warp bounded wait on the counter ahead of each GEMM launch.  With
  ``mc_stages=2`` the root instead stores chunk p (1/G of the slab) into rank p's buffer with
  unicast stores and every rank multicasts its own chunk, so that all GPUs' links carry the
  traffic; on the 8-GPU boxes this was measured slower per step (2.0-2.3 ms against 1.73 ms on
  16384^3) because every GPU's GEMM then shares its SMs with a copy kernel.  The copy kernels
  use no shared memory and few registers, so their CTAs are co-resident with the persistent
  GEMM's.  Landing buffers are double-buffered across steps; ranks acknowledge a finished step
  in the root's memory so that nothing overwrites a buffer that is still being read.
* ``chain`` (needs symmetric memory; the default where available): rank r forwards A to rank r+1 in chunks of
  ``chain_rows`` rows with copy-engine copies into the next rank's landing buffer (no SM touches the bytes), each
  followed by a flag store; a rank forwards a chunk as soon as its own copy of it has landed, so all links of the
  chain are busy at once and every hop runs at the unicast NVLink rate.  A step's forwarding is enqueued by one
  library call; the chunks alternate between ``chain_streams`` streams so that the small kernels around one copy
  run while the next copy keeps the link busy.  ``chain_fused`` (default) runs ONE gated GEMM launch per step on
  the receiving ranks, whose loaders wait inside the kernel for the chunk count of their tile's rows; without it
  there is one launch per row slab, each behind a wait for the chunks that cover the slab.
* ``nccl``: ``torch.distributed.broadcast`` per slab (any backend; used by the CPU/gloo tests).
  Its wide CTAs cannot share an SM with the GEMM's, so on 8 GPUs transfer and math serialise.

Either way the data lands in this GPU's own memory; GEMM kernels only ever read local memory.
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


def plan_slabs(m: int, shard_cols: int, k: int, *, tile_rows: int = 256, tile_cols: int = 256, in_flight: int = 74,
               gemm_tflops: float = 1350.0, bcast_gbs: float = 650.0, per_slab_us: float = 25.0,
               max_slabs: int = 16) -> List[Tuple[int, int]]:
    """Row slabs of A that minimise the modelled time of one step on a non-root rank.

    Model: the broadcast of a slab takes rows * K * 2 bytes / ``bcast_gbs`` and slabs are sent back to
    back; the GEMM of a slab starts when its broadcast has landed and the previous GEMM is done, and takes
    ceil(tiles / in_flight) waves of ``tile_rows x tile_cols`` tiles at ``gemm_tflops`` plus ``per_slab_us``
    of launch overhead.  Because the bytes sent so far depend only on the rows sent so far, "earliest
    finish of the first b row-blocks" is an exact dynamic programme over b.  The result keeps the first
    slab small when the step is compute-bound, the last slab small when it is transfer-bound, and sizes
    every slab to a whole number of tile waves.
    """
    if m <= 0:
        return []
    blocks = -(-m // tile_rows)
    tiles_n = max(1, -(-shard_cols // tile_cols))
    t_wave = in_flight * 2.0 * tile_rows * tile_cols * k / (gemm_tflops * 1e12)  # seconds per full wave
    t_block = tile_rows * k * 2.0 / (bcast_gbs * 1e9)                            # seconds to send one row-block
    overhead = per_slab_us * 1e-6
    inf = float("inf")
    # best[b][s] = earliest finish of the GEMMs of the first b blocks using s slabs
    best = [[inf] * (max_slabs + 1) for _ in range(blocks + 1)]
    prev = [[0] * (max_slabs + 1) for _ in range(blocks + 1)]
    best[0][0] = 0.0
    for b in range(blocks):
        for s_used in range(max_slabs):
            t_comp = best[b][s_used]
            if t_comp == inf:
                continue
            for nxt in range(b + 1, blocks + 1):
                landed = nxt * t_block
                waves = -(-((nxt - b) * tiles_n) // in_flight)
                done = max(t_comp, landed) + waves * t_wave + overhead
                if done < best[nxt][s_used + 1]:
                    best[nxt][s_used + 1] = done
                    prev[nxt][s_used + 1] = b
    s_best = min(range(1, max_slabs + 1), key=lambda s_: best[blocks][s_])
    cuts = []
    b, s_used = blocks, s_best
    while b > 0:
        pb = prev[b][s_used]
        cuts.append((pb, b))
        b, s_used = pb, s_used - 1
    cuts.reverse()
    return [(lo * tile_rows, min(m, hi * tile_rows)) for lo, hi in cuts]


class NShardedGemm:
    """``C[:, shard] = A @ B[shard].T`` on every rank, A living on ``root`` before the call.

    ``gemm_fn(a_slab, b_shard, c_slab)`` defaults to the CUDA GEMM of this package; tests on
    CPU ranks (gloo) pass their own to exercise the partition and the exchange.
    """

    def __init__(self, m: int, n: int, k: int, group=None, root: int = 0, slabs: int = 0,
                 gemm_fn: Optional[Callable] = None, device=None, ctx=None, transport: str = "auto",
                 push_ctas: int = 0, mc_stages: int = 1, chain_rows: int = 2048,
                 chain_fused: bool = True, chain_streams: int = 2, **plan_args):
        import torch
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.root = root
        self.m, self.n, self.k = m, n, k
        self.lo, self.hi = shard_bounds(n, self.world, self.rank)
        # slabs > 0: that many equal slabs; slabs == 0: sizes from the makespan model of plan_slabs()
        if self.world == 1:
            self.slabs = slab_bounds(m, 1)
        elif slabs > 0:
            self.slabs = slab_bounds(m, slabs)
        else:
            # every rank must cut A the same way: plan for the widest shard (rank 0's), not for its own
            widest = shard_bounds(n, self.world, 0)
            self.slabs = plan_slabs(m, widest[1] - widest[0], k, **plan_args)
        self.device = device
        self.ctx = ctx
        if gemm_fn is None:
            from .gemm import default_context
            self.ctx = ctx or default_context(torch.device(device).index if device is not None else None)
            gemm_fn = lambda a, b, c: self.ctx.gemm(a, b, out=c)  # noqa: E731
        self.gemm_fn = gemm_fn
        self._a_local = None
        self.push_ctas = push_ctas
        self.chain_rows = max(256, chain_rows // 256 * 256)  # rows of A per forwarded chunk
        # one GEMM launch per step whose loaders wait for the rows of A inside the kernel, instead of one per slab
        self.chain_fused = chain_fused
        if self.ctx is not None:  # the forwarded chunks alternate between this many streams
            self.ctx.set("chain_streams", chain_streams)
        self.mc_stages = mc_stages  # 2: root scatters chunks, every rank multicasts its own; 1: the root multicasts everything
        self.step = 0
        self.transport = "nccl"
        self._mc = None
        if self.world > 1 and transport in ("auto", "multimem", "chain") and getattr(self, "ctx", None) is not None:
            try:
                self._setup_multimem(device)
                # measured on 8 B200s, 16384^3: chain 1.20 ms per step, multimem 1.73 ms, nccl 1.98 ms
                self.transport = "multimem" if transport == "multimem" else "chain"
            except Exception:
                if transport in ("multimem", "chain"):
                    raise

    @property
    def shard_cols(self) -> int:
        return self.hi - self.lo

    def a_buffer(self, like):
        """This rank's landing buffer for A (the root uses its own A in place)."""
        import torch
        if self._mc is not None:
            return self._landing((self.step - 1) & 1 if self.step else 0)
        if self._a_local is None:
            self._a_local = torch.empty((self.m, self.k), dtype=like.dtype, device=like.device)
        return self._a_local

    # ----------------------------------------------------------- multimem transport --
    # 32-bit flag words behind the landing buffers of every rank:
    #   [0, G)    word r counts the slabs whose chunk r has been multicast (written by rank r on every GPU)
    #   [16]      slabs whose own chunk has landed here (written by the root with a unicast store)
    #   [32, 32+G) on the root: word r = steps that rank r has finished reading (acknowledgements)
    _FLAG_WORDS = 64
    _W_LANDED, _W_ACK = 16, 32

    def _setup_multimem(self, device):
        import torch
        import torch.distributed._symmetric_memory as symm_mem
        if self.world > 16:
            raise RuntimeError("multimem transport handles up to 16 GPUs")
        group = self.group if self.group is not None else self.dist.group.WORLD
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        slab_elems = self.m * self.k
        self._buf_elems = -(-slab_elems // 128) * 128  # keep the second buffer 256-byte aligned
        total = 2 * self._buf_elems + self._FLAG_WORDS * 2  # bf16 elements; flags are 32-bit = 2 elements each
        buf = symm_mem.empty(total, dtype=torch.bfloat16, device=dev)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, group.group_name)
        if not hdl.multicast_ptr:
            raise RuntimeError("no multicast mapping for the symmetric buffer")
        torch.cuda.synchronize(dev)
        hdl.barrier()
        self._mc = dict(
            buf=buf, hdl=hdl, mc_base=int(hdl.multicast_ptr), local_base=buf.data_ptr(),
            peer_base=[int(x) for x in hdl.buffer_ptrs], flags_off=2 * self._buf_elems * 2,
            push_stream=torch.cuda.Stream(device=dev), dev=dev)

    def _landing(self, parity: int):
        """This rank's landing buffer of the given step parity, as an M x K tensor."""
        mc = self._mc
        return mc["buf"][parity * self._buf_elems: parity * self._buf_elems + self.m * self.k].view(self.m, self.k)

    def _chunk(self, nbytes: int, rank: int) -> Tuple[int, int]:
        """Byte range of rank's share of a slab of nbytes (equal shares in 16-byte units, as the kernels cut it)."""
        n16 = nbytes // 16
        return n16 * rank // self.world * 16, n16 * (rank + 1) // self.world * 16

    def _run_multimem(self, a_root, b_shard, c_shard):
        """Two-stage replication per slab: the root stores chunk p of the slab into rank p's landing buffer
        (unicast), then every rank multicasts its own chunk to all ranks, so that all GPUs' links carry the
        traffic instead of the root's alone.  A GEMM waits until all G chunks of its slab are in."""
        import torch
        mc, ctx, G = self._mc, self.ctx, self.world
        n_slabs = len(self.slabs)
        parity = self.step & 1
        base = self.step * n_slabs
        par_off = parity * self._buf_elems * 2
        flags_mc = mc["mc_base"] + mc["flags_off"]
        flags_local = mc["local_base"] + mc["flags_off"]
        row_bytes = self.k * 2
        cur = torch.cuda.current_stream(mc["dev"])
        push = mc["push_stream"]
        is_root = self.rank == self.root
        if is_root:
            push.wait_stream(cur)  # A may have been produced by earlier work of the caller's stream
            if self.step >= 2:
                # the buffer of this parity was last read in step - 2: every rank must have acknowledged it
                ctx.flags_wait(flags_local + self._W_ACK * 4, G, self.step - 1, stream=push)
        for i, (lo, hi) in enumerate(self.slabs):
            nbytes = (hi - lo) * row_bytes
            off = par_off + lo * row_bytes
            c_lo, c_hi = self._chunk(nbytes, self.rank)
            value = base + i + 1
            if self.mc_stages == 1:
                if is_root:
                    ctx.mc_push(a_root.data_ptr() + lo * row_bytes, mc["mc_base"] + off, nbytes,
                                flags_mc + self.rank * 4, value, ctas=self.push_ctas, stream=push)
                continue
            if is_root:
                ctx.scatter_push(a_root.data_ptr() + lo * row_bytes, [pb + off for pb in mc["peer_base"]],
                                 [pb + mc["flags_off"] + self._W_LANDED * 4 for pb in mc["peer_base"]], self.root,
                                 nbytes, value, ctas=self.push_ctas, stream=push)
                if c_hi > c_lo:
                    ctx.mc_push(a_root.data_ptr() + lo * row_bytes + c_lo, mc["mc_base"] + off + c_lo, c_hi - c_lo,
                                flags_mc + self.rank * 4, value, ctas=self.push_ctas, stream=push)
                else:
                    ctx.flag_store(flags_mc + self.rank * 4, value, stream=push)
            else:
                ctx.mc_push_after(flags_local + self._W_LANDED * 4, value, mc["local_base"] + off + c_lo,
                                  mc["mc_base"] + off + c_lo, max(c_hi - c_lo, 0), flags_mc + self.rank * 4, value,
                                  ctas=self.push_ctas, stream=push)
        a = a_root if is_root else self._landing(parity)
        for i, (lo, hi) in enumerate(self.slabs):
            if not is_root and self.mc_stages == 1:
                ctx.flags_wait(flags_local + self.root * 4, 1, base + i + 1, stream=cur)
            elif not is_root:
                ctx.flags_wait(flags_local, G, base + i + 1, stream=cur)
            self.gemm_fn(a[lo:hi], b_shard, c_shard[lo:hi])
        if is_root:
            cur.wait_stream(push)  # A must not change before the pushes have read it
        ctx.flag_store(mc["peer_base"][self.root] + mc["flags_off"] + (self._W_ACK + self.rank) * 4, self.step + 1,
                       stream=cur)
        self.step += 1
        return c_shard

    def _run_chain(self, a_root, b_shard, c_shard, a_ready=None):
        """Rank r receives chunks from r - 1 and forwards them to r + 1 with copy-engine copies; the flag word
        LANDED of a rank counts the chunks that have arrived there.  Ranks are chained in rank order from the root
        (the root must be rank 0).

        Streams.  The forwarding of a step is enqueued on a helper stream with one library call
        (``maize_chain_forward``); the GEMM on the caller's stream.  What the helper stream has to wait for before it
        may read A on the root: ``a_ready`` (a CUDA event after which A is valid) when given, else everything the
        caller's stream holds so far.  With an event, the replication of step s + 1 runs while step s still
        multiplies (the landing buffers are double-buffered and a rank's buffer is only overwritten after that rank
        has acknowledged the step that used it), so that back-to-back steps are bound by the slower of transfer and
        math instead of their sum.  The receiving ranks' forwarding never depends on their compute stream."""
        import torch
        mc, ctx, G = self._mc, self.ctx, self.world
        if self.root != 0:
            raise RuntimeError("the chain transport expects the root to be rank 0")
        chunks = [(lo, min(self.m, lo + self.chain_rows)) for lo in range(0, self.m, self.chain_rows)]
        C = len(chunks)
        parity = self.step & 1
        base = self.step * C
        par_off = parity * self._buf_elems * 2
        row_bytes = self.k * 2
        flags_local = mc["local_base"] + mc["flags_off"]
        cur = torch.cuda.current_stream(mc["dev"])
        push = mc["push_stream"]
        r = self.rank
        last = r == G - 1
        if not last:
            nxt = mc["peer_base"][r + 1]
            if r == 0:
                if a_ready is not None:
                    push.wait_event(a_ready)
                else:
                    push.wait_stream(cur)  # A may come from earlier work of the caller's stream
            if self.step >= 2:
                # the next rank's buffer of this parity was last used in step - 2
                ctx.flags_wait(flags_local + self._W_ACK * 4, 1, self.step - 1, stream=push)
            src_base = a_root.data_ptr() if r == 0 else mc["local_base"] + par_off
            ctx.chain_forward(None if r == 0 else flags_local + self._W_LANDED * 4, base + 1, nxt + par_off, src_base,
                              self.m * row_bytes, self.chain_rows * row_bytes,
                              nxt + mc["flags_off"] + self._W_LANDED * 4, stream=push)
        a = a_root if r == 0 else self._landing(parity)
        if self.chain_fused:
            if r == 0:
                self.gemm_fn(a, b_shard, c_shard)
            else:
                ctx.gemm_gated(a, b_shard, c_shard, flags_local + self._W_LANDED * 4, base, self.chain_rows, stream=cur)
        for lo, hi in (self.slabs if not self.chain_fused else []):
            if r != 0:
                need = next(i for i, (c_lo, c_hi) in enumerate(chunks) if c_hi >= hi)  # last chunk covering the slab
                ctx.flags_wait(flags_local + self._W_LANDED * 4, 1, base + need + 1, stream=cur)
            self.gemm_fn(a[lo:hi], b_shard, c_shard[lo:hi])
        if not last:
            cur.wait_stream(push)  # this rank's copy of A must stay until it has been forwarded
        if r != 0:
            # tell the previous rank that this step's buffer has been read (by the GEMMs and by the forwarding)
            ctx.flag_store(mc["peer_base"][r - 1] + mc["flags_off"] + self._W_ACK * 4, self.step + 1, stream=cur)
        self.step += 1
        return c_shard

    def gather_c(self, c_shard):
        """Dense M x N matrix C on every rank from the column blocks (for callers that do not want C sharded).
        The hot path keeps C sharded; this is a convenience on top of ``all_gather``."""
        import torch
        if self.world == 1:
            return c_shard
        widest = shard_bounds(self.n, self.world, 0)
        width = widest[1] - widest[0]
        padded = c_shard
        if c_shard.shape[1] != width:
            padded = torch.zeros((self.m, width), dtype=c_shard.dtype, device=c_shard.device)
            padded[:, :c_shard.shape[1]] = c_shard
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        self.dist.all_gather(parts, padded.contiguous(), group=self.group)
        cols = [parts[r][:, :shard_bounds(self.n, self.world, r)[1] - shard_bounds(self.n, self.world, r)[0]]
                for r in range(self.world)]
        return torch.cat(cols, dim=1)

    def run(self, a_root, b_shard, c_shard, a_ready=None):
        """One step: replicate A from the root and multiply as its rows arrive.

        ``a_root`` is the M x K matrix on the root and ignored elsewhere (may be None);
        ``b_shard`` is this rank's (hi-lo) x K block of B; ``c_shard`` is M x (hi-lo).
        ``a_ready`` (root, chain transport): a ``torch.cuda.Event`` after which ``a_root`` holds this step's A.
        Without it the replication waits for everything the current stream holds, the previous step's GEMM
        included; with it, the replication of a step overlaps the previous step's math.
        """
        if self.world == 1:
            self.gemm_fn(a_root, b_shard, c_shard)
            return c_shard
        if self.transport == "multimem":
            return self._run_multimem(a_root, b_shard, c_shard)
        if self.transport == "chain":
            return self._run_chain(a_root, b_shard, c_shard, a_ready)
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
