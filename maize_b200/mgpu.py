"""One host process driving several GPUs: the N-sharded GEMM through ``maize_mgpu_*`` of the C ABI.

Where ``maize_b200.sharded`` runs one process per GPU over ``torch.distributed``, this binds the single-process
form a compiled caller of the library would use (the reference's GEMM entry point,
crates/maize_tile/src/gemm/mod.rs:37-55, is called from one host thread): device ``g`` of the list owns a
contiguous block of rows of B and the matching column block of C, A is forwarded from the root along a chain of
peer copies.  torch is used for device memory only; the handle has its own streams, so tensors produced on
torch's streams must be complete (``torch.cuda.synchronize``) before they are handed over, or be produced on
``stream(index)``.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

from . import _ffi
from .gemm import MaizeError


class MultiGpu:
    def __init__(self, devices: Sequence[int]):
        self._lib = _ffi.load()
        self.devices = [int(d) for d in devices]
        arr = (ctypes.c_int * len(self.devices))(*self.devices)
        handle = ctypes.c_void_p()
        st = self._lib.maize_mgpu_create(len(self.devices), arr, ctypes.byref(handle))
        if st != _ffi.OK:
            raise MaizeError(st, self._lib.maize_status_string(st).decode())
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.maize_mgpu_destroy(self._h)
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

    def _check(self, st: int) -> None:
        if st != _ffi.OK:
            raise MaizeError(st, self._lib.maize_mgpu_last_error(self._h).decode())

    def __len__(self) -> int:
        return int(self._lib.maize_mgpu_size(self._h))

    def set(self, key: str, value: int) -> None:
        self._check(self._lib.maize_mgpu_set(self._h, key.encode(), int(value)))

    def stream(self, index: int) -> int:
        """The cudaStream_t (as an integer) on which device ``index``'s GEMMs run."""
        return int(self._lib.maize_mgpu_stream(self._h, index) or 0)

    def shard(self, n_rows: int, index: int) -> Tuple[int, int]:
        """Rows [first, end) of B / columns of C that device ``index`` owns."""
        lo, hi = ctypes.c_uint32(), ctypes.c_uint32()
        self._check(self._lib.maize_mgpu_shard(self._h, n_rows, index, ctypes.byref(lo), ctypes.byref(hi)))
        return lo.value, hi.value

    def gemm_nsharded(self, root: int, a_root, a_local: List, b_shards: List, c_shards: List, n: int) -> None:
        """Enqueue one step on device tensors: ``a_root`` is M x K on device ``root``; ``a_local[g]`` an M x K landing
        buffer on device g (None for the root); ``b_shards[g]`` / ``c_shards[g]`` device g's blocks.  Returns when
        enqueued; ``sync()`` waits."""
        m, k = a_root.shape
        G = len(self.devices)

        def ptrs(ts):
            return (ctypes.c_void_p * G)(*[ctypes.c_void_p(t.data_ptr() if t is not None else None) for t in ts])

        for t in [a_root, *a_local, *b_shards, *c_shards]:
            if t is not None and not t.is_contiguous():
                raise MaizeError(_ffi.INVALID_ARG, "the multi-GPU entry point takes dense tensors")
        self._check(self._lib.maize_gemm_bf16_nsharded(self._h, root, a_root.data_ptr(), m, k, ptrs(a_local),
                                                       ptrs(b_shards), n, ptrs(c_shards)))

    def gemm_nsharded_host(self, root: int, a_ptr: int, m: int, k: int, b_ptr: int, n: int, c_ptr: int) -> None:
        """Host buffers in and out (raw addresses); copies and the wait are inside the call."""
        self._check(self._lib.maize_gemm_bf16_nsharded_host(self._h, root, a_ptr, m, k, b_ptr, n, c_ptr))

    def sync(self) -> None:
        """Wait for every device and raise if a device wait timed out."""
        self._check(self._lib.maize_mgpu_sync(self._h))
