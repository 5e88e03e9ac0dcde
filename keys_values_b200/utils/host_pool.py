"""Pinned host memory pool (native: ``csrc/host_pool.cpp``).

``HostPool(nbytes)`` takes one pinned slab; ``pool.empty(shape, dtype)`` returns a CPU tensor that views a range
of it (and gives the range back when the tensor is garbage collected or :meth:`HostPool.release` is called), so
per-step staging buffers cost microseconds instead of a ``cudaHostAlloc`` each. Tensors from the pool answer
``is_pinned() == True`` on a machine with a GPU, hence ``copy_(…, non_blocking=True)`` is truly asynchronous.
Without a GPU (or with ``pinned=False``) the slab is pageable: same interface, same allocator.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, Optional, Sequence

import torch

from keys_values_b200.ops import cuda as _cu

_TOO_LARGE = -7


class HostPool:
    def __init__(self, nbytes: int, pinned: Optional[bool] = None):
        if pinned is None:
            pinned = torch.cuda.is_available()
        self.pinned = bool(pinned)
        self._lib = _cu.lib()
        handle = ctypes.c_void_p()
        _cu._check(self._lib.kvb_host_pool_create(ctypes.byref(handle), ctypes.c_longlong(nbytes), int(self.pinned)), "host_pool_create")
        self._handle = handle
        self._live: Dict[int, int] = {}  # pointer -> bytes of the ranges handed out
        self.fallbacks = 0               # requests that did not fit and went to the ordinary allocator

    # ------------------------------------------------------------------ tensors
    def empty(self, shape: Sequence[int], dtype: torch.dtype = torch.uint8) -> torch.Tensor:
        """Uninitialised CPU tensor inside the pool; falls back to an ordinary (pinned, if the pool is) tensor
        when no free range fits."""
        shape = tuple(int(x) for x in shape)
        numel = 1
        for x in shape:
            numel *= x
        nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 1)
        ptr = ctypes.c_void_p()
        rc = self._lib.kvb_host_pool_alloc(self._handle, ctypes.c_longlong(nbytes), ctypes.byref(ptr))
        if rc == _TOO_LARGE:
            self.fallbacks += 1
            return torch.empty(shape, dtype=dtype, pin_memory=self.pinned and torch.cuda.is_available())
        _cu._check(rc, "host_pool_alloc")
        addr = ptr.value
        buf = (ctypes.c_uint8 * nbytes).from_address(addr)
        t = torch.frombuffer(buf, dtype=torch.uint8, count=nbytes)[: numel * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)
        self._live[addr] = nbytes
        # the range returns to the pool when the last view of this storage is gone
        weakref.finalize(buf, HostPool._release_addr, weakref.ref(self), addr)  # torch keeps `buf` alive as long as the storage
        return t

    @staticmethod
    def _release_addr(pool_ref, addr: int) -> None:
        pool = pool_ref()
        if pool is not None and addr in pool._live and pool._handle:
            pool._live.pop(addr)
            pool._lib.kvb_host_pool_free(pool._handle, ctypes.c_void_p(addr))

    def release(self, tensor: torch.Tensor) -> None:
        """Give the range of ``tensor`` back now (the tensor must not be used afterwards)."""
        HostPool._release_addr(weakref.ref(self), tensor.untyped_storage().data_ptr())

    # ------------------------------------------------------------------- queries
    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * 6)()
        _cu._check(self._lib.kvb_host_pool_stats(self._handle, out), "host_pool_stats")
        keys = ("capacity", "in_use", "peak", "largest_free", "allocations", "failures")
        return dict(zip(keys, (int(v) for v in out)), fallbacks=self.fallbacks)

    def close(self) -> None:
        if self._handle:
            self._live.clear()
            self._lib.kvb_host_pool_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            if not self._live:
                self.close()
        except Exception:
            pass


_DEFAULT: Optional[HostPool] = None


def default_pool() -> Optional[HostPool]:
    """The process-wide pool for staging buffers of the offload paths (checkpoints, streamed weights' gradients):
    created on first use with ``KVB200_HOST_POOL_GB`` gigabytes (default 8; 0 switches it off) of pinned memory on a
    machine with a GPU. Requests that do not fit fall back to ordinary pinned tensors."""
    global _DEFAULT
    import os

    if _DEFAULT is None:
        gb = float(os.environ.get("KVB200_HOST_POOL_GB", "8"))
        if gb <= 0 or not torch.cuda.is_available():
            return None
        try:
            _DEFAULT = HostPool(int(gb * 2**30), pinned=True)
        except Exception:
            os.environ["KVB200_HOST_POOL_GB"] = "0"  # the host cannot pin that much: ordinary pinned tensors from now on
            return None
    return _DEFAULT


def pinned_empty(shape, dtype) -> torch.Tensor:
    """Pinned (where a GPU is present) uninitialised host tensor, from the default pool when it has room."""
    pool = default_pool()
    if pool is not None:
        return pool.empty(shape, dtype)
    return torch.empty(tuple(shape), dtype=dtype, pin_memory=torch.cuda.is_available())
