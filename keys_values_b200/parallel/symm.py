"""Symmetric memory over NVLink: one arena per rank, mapped into every rank.

Each rank allocates ``numel`` elements (plus a small flag area) with ``cudaMalloc``,
publishes a CUDA IPC handle, and maps the arenas of all peers of the same node.
The handles travel over ``torch.distributed`` (``all_gather_object``), which is the
only use of the process group here; the data path is the kernels of
``csrc/comm.cu`` that read and write the peers' arenas directly.

The reference has no counterpart: its only collective is NCCL ``all_reduce`` through
Lightning Fabric (``keys_values/optimize/grad_accumulate.py:24-82``).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from keys_values_b200.ops import cuda as _cu

FLAG_BYTES = 256


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None,
        }


class SymmetricArena:
    def __init__(self, numel: int, dtype: torch.dtype, device, world_size: int, rank: int, group=None,
                 timeout_s: float = 20.0, n_ctas: int = 0):
        self.numel, self.dtype = numel, dtype
        self.device = torch.device(device)
        self.world_size, self.rank, self.group = world_size, rank, group
        self.timeout_s, self.n_ctas = timeout_s, n_ctas
        lib = _cu.lib()
        esize = torch.empty((), dtype=dtype).element_size()
        self.data_bytes = (numel * esize + 255) // 256 * 256
        self.total_bytes = self.data_bytes + FLAG_BYTES
        torch.cuda.set_device(self.device)
        ptr = ctypes.c_void_p()
        _cu._check(lib.kvb_symm_alloc(ctypes.byref(ptr), ctypes.c_longlong(self.total_bytes)), "symm_alloc")
        self._ptr = ptr.value
        self._raw = _RawCudaBuffer(self._ptr, self.total_bytes)
        whole = torch.as_tensor(self._raw, device=self.device)
        self.tensor = whole[: numel * esize].view(dtype)
        # exchange IPC handles
        hsize = lib.kvb_ipc_handle_size()
        hbuf = (ctypes.c_ubyte * hsize)()
        _cu._check(lib.kvb_ipc_get_handle(ctypes.c_void_p(self._ptr), hbuf), "ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * world_size
        dist.all_gather_object(handles, bytes(hbuf), group=group)
        self._peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self._peer_ptrs.append(self._ptr)
                continue
            out = ctypes.c_void_p()
            hb = (ctypes.c_ubyte * hsize).from_buffer_copy(h)
            _cu._check(lib.kvb_ipc_open_handle(hb, ctypes.byref(out)), "ipc_open_handle")
            self._peer_ptrs.append(out.value)
            self._opened.append(out.value)
        self._bases = (ctypes.c_void_p * world_size)(*self._peer_ptrs)
        self._flags = (ctypes.c_void_p * world_size)(*[p + self.data_bytes for p in self._peer_ptrs])
        self._sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._epoch = 1
        self._dtype_code = _cu._code(dtype)
        dist.barrier(group=group)

    def all_reduce_mean_(self, start: int = 0, end: Optional[int] = None, scale: Optional[float] = None) -> None:
        """In-place mean over ranks of ``tensor[start:end]`` on the current stream. All ranks
        must call this with the same arguments, in the same order."""
        end = self.numel if end is None else end
        align = 16 // self.tensor.element_size()
        start_a = start // align * align
        end_a = min((end + align - 1) // align * align, (self.numel + align - 1) // align * align)
        count = end_a - start_a
        if count <= 0:
            return
        st = _cu.status_word(self.device)
        sc = 1.0 / self.world_size if scale is None else scale
        _cu._check(
            _cu.lib().kvb_allreduce_mean(
                self._bases, self._flags, self.rank, self.world_size, ctypes.c_longlong(start_a), ctypes.c_longlong(count),
                ctypes.c_float(sc), ctypes.c_uint(self._epoch), ctypes.c_void_p(self._sync.data_ptr()), self._dtype_code,
                self.n_ctas, ctypes.c_void_p(st.data_ptr()), ctypes.c_double(self.timeout_s),
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream),
            ),
            "allreduce_mean",
        )
        self._epoch += 3
        _cu._count()

    def reset_sync(self) -> None:
        """After a wait that ran out: the kernel left its grid-barrier words and this rank's flags in a
        state of the abandoned launch. Clear them so that a later launch (after the ranks have agreed to go
        on) does not see stale arrivals. Every rank that goes on must call this."""
        self._sync.zero_()
        esize = torch.empty((), dtype=self.dtype).element_size()
        whole = torch.as_tensor(self._raw, device=self.device)
        whole[self.data_bytes : self.data_bytes + FLAG_BYTES].zero_()
        self._epoch = 1
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        lib = _cu.lib()
        for p in self._opened:
            lib.kvb_ipc_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self._ptr:
            self.tensor = None
            lib.kvb_symm_free(ctypes.c_void_p(self._ptr))
            self._ptr = 0
