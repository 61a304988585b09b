"""Host-side mirror of the reference's GEMM call shape over the C ABI.

The reference builds its GEMM from ``Matrix::new(ptr, nrows, ncols)`` pairs
(crates/maize_tile/src/gmem/matrix.rs:13-18, src/main.rs:46-48) handed to
``sm80_gemm_smem_multibuffer`` (crates/maize_tile/src/gemm/mod.rs:37-90).  The
same shape is kept: ``Matrix`` is {ptr, nrows, ncols}; ``Context.gemm`` takes A
(M x K), B (N x K, K-major) and C (M x N) and launches the sm_100a kernels.
torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

from . import _ffi


class MaizeError(RuntimeError):
    def __init__(self, status: int, message: str = ""):
        self.status = status
        name = _ffi.STATUS_NAMES.get(status, f"status {status}")
        super().__init__(f"{name}: {message}" if message else name)


@dataclass(frozen=True)
class Matrix:
    """{ptr, nrows, ncols} of a dense row-major bf16 matrix in device memory."""
    ptr: int
    nrows: int
    ncols: int

    @classmethod
    def new(cls, ptr: int, nrows: int, ncols: int) -> "Matrix":
        return cls(int(ptr), int(nrows), int(ncols))

    @classmethod
    def from_tensor(cls, t) -> "Matrix":
        import torch
        if t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise MaizeError(_ffi.INVALID_ARG, "expected a contiguous 2-D bfloat16 tensor")
        return cls(t.data_ptr(), t.shape[0], t.shape[1])

    def as_c(self) -> _ffi.GlobalMatrix:
        return _ffi.GlobalMatrix(self.ptr, self.nrows, self.ncols)


def _stream_handle(stream) -> Optional[int]:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Context:
    """One per host thread / stream; owns the device status word and tunables."""

    def __init__(self, device: int = 0):
        self._lib = _ffi.load()
        handle = ctypes.c_void_p()
        st = self._lib.maize_ctx_create(int(device), ctypes.byref(handle))
        if st != _ffi.OK:
            raise MaizeError(st, self._lib.maize_status_string(st).decode())
        self._h = handle
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.maize_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------ helpers --
    def _check(self, st: int) -> None:
        if st != _ffi.OK:
            raise MaizeError(st, self._lib.maize_last_error(self._h).decode())

    def set(self, key: str, value: int) -> None:
        self._check(self._lib.maize_ctx_set(self._h, key.encode(), int(value)))

    def get(self, key: str) -> int:
        out = ctypes.c_int64()
        self._check(self._lib.maize_ctx_get(self._h, key.encode(), ctypes.byref(out)))
        return out.value

    @property
    def launch_count(self) -> int:
        return int(self._lib.maize_ctx_launch_count(self._h))

    def pick_kernel(self, m: int, n: int, k: int) -> str:
        return self._lib.maize_kernel_name(self._lib.maize_pick_kernel(self._h, m, n, k)).decode()

    @property
    def last_kernel(self) -> str:
        """Name of the GEMM kernel the last call on this context launched ("" before the first)."""
        kid = self.get("last_kernel")
        return self._lib.maize_kernel_name(kid).decode() if kid > 0 else ""

    def poll(self, stream=None) -> None:
        """Synchronise the stream and raise if a device wait timed out."""
        self._check(self._lib.maize_ctx_poll(self._h, _stream_handle(stream)))

    # --------------------------------------------------------------- GEMM --
    def gemm_matrices(self, a: Matrix, b: Matrix, c: Matrix, stream=None) -> None:
        """C = A @ B.T through the {ptr, nrows, ncols} bundles."""
        ca, cb, cc = a.as_c(), b.as_c(), c.as_c()
        self._check(self._lib.maize_gemm_bf16_m(self._h, ctypes.byref(ca), ctypes.byref(cb), ctypes.byref(cc),
                                                _stream_handle(stream)))

    def gemm_raw(self, a_ptr, a_rows, a_cols, b_ptr, b_rows, b_cols, c_ptr, c_rows, c_cols, stream=None) -> None:
        self._check(self._lib.maize_gemm_bf16(self._h, a_ptr, a_rows, a_cols, b_ptr, b_rows, b_cols, c_ptr, c_rows,
                                              c_cols, _stream_handle(stream)))

    def gemm_ld(self, a_ptr, lda, b_ptr, ldb, c_ptr, ldc, m, n, k, stream=None) -> None:
        self._check(self._lib.maize_gemm_bf16_ld(self._h, a_ptr, lda, b_ptr, ldb, c_ptr, ldc, m, n, k,
                                                 _stream_handle(stream)))

    def gemm_host(self, a_ptr, a_rows, a_cols, b_ptr, b_rows, b_cols, c_ptr, c_rows, c_cols, stream=None) -> None:
        """Host buffers in, host buffer out; copies and the wait are inside the call."""
        self._check(self._lib.maize_gemm_bf16_host(self._h, a_ptr, a_rows, a_cols, b_ptr, b_rows, b_cols, c_ptr,
                                                   c_rows, c_cols, _stream_handle(stream)))

    def gemm(self, a, b, out=None, stream=None):
        """``out = a @ b.T`` for bf16 CUDA tensors: a is M x K, b is N x K; rows may be strided."""
        import torch
        for name, t in (("a", a), ("b", b)):
            if t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_cuda or (t.shape[1] > 1 and t.stride(1) != 1):
                raise MaizeError(_ffi.INVALID_ARG, f"{name}: expected a 2-D bfloat16 CUDA tensor with unit column stride")
        m, k = a.shape
        n, kb = b.shape
        if k != kb:
            raise MaizeError(_ffi.INVALID_ARG, "a.shape[1] != b.shape[1] (b is stored N x K)")
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
        elif out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_cuda or (n > 1 and out.stride(1) != 1):
            raise MaizeError(_ffi.INVALID_ARG, "out: expected an M x N bfloat16 CUDA tensor with unit column stride")
        lda = a.stride(0) if m > 1 else max(k, 1)
        ldb = b.stride(0) if n > 1 else max(k, 1)
        ldc = out.stride(0) if m > 1 else max(n, 1)
        self.gemm_ld(a.data_ptr(), lda, b.data_ptr(), ldb, out.data_ptr(), ldc, m, n, k, stream)
        return out

    def gemm_gated(self, a, b, out, rows_landed_ptr: int, landed_base: int, rows_per_count: int, stream=None):
        """``out = a @ b.T`` for an ``a`` whose rows are still arriving in row order: the kernel reads rows
        [0, r) only once the 32-bit word at ``rows_landed_ptr`` has reached landed_base + ceil(r / rows_per_count).
        The wait is bounded ("timeout_ns"); ``poll()`` reports a count that never came as a timeout."""
        m, k = a.shape
        n = b.shape[0]
        if b.shape[1] != k or tuple(out.shape) != (m, n):
            raise MaizeError(_ffi.INVALID_ARG, "gemm_gated: a is M x K, b is N x K, out is M x N")
        lda = a.stride(0) if m > 1 else max(k, 1)
        ldb = b.stride(0) if n > 1 else max(k, 1)
        ldc = out.stride(0) if m > 1 else max(n, 1)
        self._check(self._lib.maize_gemm_bf16_gated(self._h, a.data_ptr(), lda, b.data_ptr(), ldb, out.data_ptr(), ldc,
                                                    m, n, k, rows_landed_ptr, landed_base & 0xFFFFFFFF, rows_per_count,
                                                    _stream_handle(stream)))
        return out

    PROFILE_SLOTS = ("producer_wait_empty", "mma_wait_full", "mma_wait_acc_empty", "epilogue_wait_acc_full",
                     "epilogue_drain", "cta_cycles", "tiles", "spare")

    def read_profile(self, stream=None):
        """Per-CTA cycle counters of the last launch (after ``set("profile", 1)``): list of dicts."""
        buf = (ctypes.c_uint64 * (8 * 1024))()
        n = self._lib.maize_ctx_read_profile(self._h, buf, 1024, _stream_handle(stream))
        return [dict(zip(self.PROFILE_SLOTS, buf[8 * i:8 * i + 8])) for i in range(n)]

    # ------------------------------------------------- multi-GPU building blocks --
    def mc_push(self, src_ptr: int, mc_dst_ptr: int, nbytes: int, mc_flag_ptr: int, flag_value: int, ctas: int = 0,
                stream=None) -> None:
        """Push local bytes to every GPU's replica through the multicast address, then publish a flag value."""
        self._check(self._lib.maize_mc_push(self._h, src_ptr, mc_dst_ptr, nbytes, mc_flag_ptr, flag_value & 0xFFFFFFFF,
                                            ctas, _stream_handle(stream)))

    def mc_push_after(self, wait_flag_ptr: int, wait_value: int, src_ptr: int, mc_dst_ptr: int, nbytes: int,
                      mc_flag_ptr: int, flag_value: int, ctas: int = 0, stream=None) -> None:
        """Like mc_push, but the kernel first waits for the local word at wait_flag_ptr to reach wait_value."""
        self._check(self._lib.maize_mc_push_after(self._h, wait_flag_ptr, wait_value & 0xFFFFFFFF, src_ptr, mc_dst_ptr,
                                                  nbytes, mc_flag_ptr, flag_value & 0xFFFFFFFF, ctas,
                                                  _stream_handle(stream)))

    def scatter_push(self, src_ptr: int, peer_dst_ptrs, peer_flag_ptrs, root: int, nbytes: int, flag_value: int,
                     ctas: int = 0, stream=None) -> None:
        """Root: store chunk p of the source into rank p's landing buffer and publish a flag there."""
        world = len(peer_dst_ptrs)
        dst = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in peer_dst_ptrs])
        flg = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in peer_flag_ptrs])
        self._check(self._lib.maize_scatter_push(self._h, src_ptr, dst, flg, world, root, nbytes,
                                                 flag_value & 0xFFFFFFFF, ctas, _stream_handle(stream)))

    def copy_async(self, dst_ptr: int, src_ptr: int, nbytes: int, stream=None) -> None:
        """Device-to-device copy on the copy engines; dst may be a peer-mapped address."""
        self._check(self._lib.maize_copy_async(self._h, dst_ptr, src_ptr, nbytes, _stream_handle(stream)))

    def chain_forward(self, wait_flag_ptr, first_value: int, dst_ptr: int, src_ptr: int, total_bytes: int,
                      chunk_bytes: int, dst_flag_ptr: int, stream=None) -> None:
        """Enqueue (wait for chunk i, copy it to the next rank, publish i) for every chunk of a step in one call."""
        self._check(self._lib.maize_chain_forward(self._h, wait_flag_ptr, first_value & 0xFFFFFFFF, dst_ptr, src_ptr,
                                                  total_bytes, chunk_bytes, dst_flag_ptr, _stream_handle(stream)))

    def flags_wait(self, flags_ptr: int, count: int, value: int, stream=None) -> None:
        self._check(self._lib.maize_flags_wait(self._h, flags_ptr, count, value & 0xFFFFFFFF, _stream_handle(stream)))

    def flag_store(self, flag_ptr: int, value: int, stream=None) -> None:
        self._check(self._lib.maize_flag_store(self._h, flag_ptr, value & 0xFFFFFFFF, _stream_handle(stream)))

    def gemm_kn(self, a, b, out=None, stream=None):
        """``out = a @ b`` for bf16 CUDA tensors with b given K x N (N contiguous), the layout the reference's
        demo walks; rows may be strided."""
        import torch
        for name, t in (("a", a), ("b", b)):
            if t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_cuda or (t.shape[1] > 1 and t.stride(1) != 1):
                raise MaizeError(_ffi.INVALID_ARG, f"{name}: expected a 2-D bfloat16 CUDA tensor with unit column stride")
        m, k = a.shape
        kb, n = b.shape
        if k != kb:
            raise MaizeError(_ffi.INVALID_ARG, "a.shape[1] != b.shape[0] (b is stored K x N)")
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
        elif out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_cuda or (n > 1 and out.stride(1) != 1):
            raise MaizeError(_ffi.INVALID_ARG, "out: expected an M x N bfloat16 CUDA tensor with unit column stride")
        lda = a.stride(0) if m > 1 else max(k, 8)
        ldb = b.stride(0) if k > 1 else max(n, 8)
        ldc = out.stride(0) if m > 1 else max(n, 1)
        self._check(self._lib.maize_gemm_bf16_kn_ld(self._h, a.data_ptr(), lda, b.data_ptr(), ldb, out.data_ptr(), ldc,
                                                    m, n, k, _stream_handle(stream)))
        return out

    def debug_wait_expires(self, budget_ns: int, stream=None) -> None:
        self._check(self._lib.maize_debug_wait_expires(self._h, int(budget_ns), _stream_handle(stream)))


_default_ctx = {}


def default_context(device: Optional[int] = None) -> Context:
    import torch
    if device is None:
        device = torch.cuda.current_device()
    ctx = _default_ctx.get(device)
    if ctx is None:
        ctx = _default_ctx[device] = Context(device)
    return ctx


def gemm(a, b, out=None, stream=None):
    """``a @ b.T`` on the B200 kernels (module-level convenience over a cached Context)."""
    return default_context(a.device.index).gemm(a, b, out=out, stream=stream)


def gemm_skinny_static(a, b, out, stream=None, device_status=None):
    """``out = a @ b.T`` for M <= 32 through the entry point that allocates nothing.

    For callers that may not allocate device memory at this point (so ``out`` must be passed in): the
    kernel's scratch is a fixed array inside the library (8 MiB per GPU).  Shapes beyond what that array
    can serve raise ``MaizeError(UNSUPPORTED)`` with the sizes in the message.  Calls that could overlap
    on the GPU share the array and must be ordered by the caller.  ``device_status``: optional int32[4]
    CUDA tensor that receives a timeout code.
    """
    import torch
    lib = _ffi.load()
    err = ctypes.create_string_buffer(256)
    # the C entry assumes dense rows (lda = ldb = K, ldc = N) on the current device: check before handing out pointers
    cur = torch.cuda.current_device()
    for name, t in (("a", a), ("b", b), ("out", out)):
        if (t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_cuda or t.device.index != cur
                or (t.shape[1] > 1 and t.stride(1) != 1) or (t.shape[0] > 1 and t.stride(0) != t.shape[1])):
            raise MaizeError(_ffi.INVALID_ARG, f"{name}: expected a dense 2-D bfloat16 tensor on the current CUDA device")
    if device_status is not None and (device_status.dtype != torch.int32 or device_status.numel() < 4
                                      or not device_status.is_cuda or not device_status.is_contiguous()):
        raise MaizeError(_ffi.INVALID_ARG, "device_status: expected a contiguous int32 CUDA tensor of at least 4 elements")
    m, k = a.shape
    n, kb = b.shape
    st = lib.maize_gemm_bf16_skinny_static(a.data_ptr(), m, k, b.data_ptr(), n, kb, out.data_ptr(), out.shape[0],
                                           out.shape[1], _stream_handle(stream),
                                           device_status.data_ptr() if device_status is not None else None,
                                           err, len(err))
    if st != _ffi.OK:
        raise MaizeError(st, err.value.decode())
    return out
