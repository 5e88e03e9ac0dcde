"""Storage of keys and values, independent of the cache policy.

Parity: ``keys_values/kvcache/buffers.py:31-619``. Buffers have shape
``(max_batch_size, n_query_groups, cache_length, head_size)`` and are allocated
lazily on first use, so that they can be deallocated between the forward and the
backward pass of a training step and share device memory with it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from keys_values_b200 import ops
from keys_values_b200.attention.base import DefaultKeysAndValues, KeysAndValues
from keys_values_b200.kvcache.base import KVCacheParams, bits_for_torch_dtype


@dataclass(frozen=True)
class KVCacheBuffersParams:
    max_batch_size: int
    n_query_groups: int
    head_size: int
    dtype: Optional[torch.dtype] = None
    device: Optional[torch.device] = None

    @staticmethod
    def from_params(params: KVCacheParams, device=None) -> "KVCacheBuffersParams":
        return KVCacheBuffersParams(params.max_batch_size, params.n_query_groups, params.head_size, params.dtype, device)


def positions_wrap_around(num: int, current: int, start: int, end: int, batch_size: int, n_query_groups: int, device, return_tensor=True):
    """Slots for ``num`` new entries of a ring buffer over ``[start, end)`` whose
    next free position is ``current``. Returns ``(B, G, num)`` int32 positions."""
    if not (start <= current < end):
        raise ValueError(f"need start={start} <= current={current} < end={end}")
    width = end - start
    if num > width:
        raise ValueError(f"num={num} exceeds ring width {width}")
    pos = (torch.arange(num, device=device, dtype=torch.int32) + (current - start)) % width + start
    return pos.view(1, 1, num).expand(batch_size, n_query_groups, num)


class KVCacheBuffers(torch.nn.Module):
    def __init__(self, params: KVCacheBuffersParams, cache_length: int):
        super().__init__()
        self.params = params
        self.cache_length = cache_length
        self.current_length = 0
        self.batch_size: Optional[int] = None
        # set by the cache around a single-token step that is served by the decode kernel
        self.decode_mode = False

    def supports_direct_decode(self) -> bool:
        return False

    def decode_attention(self, query: torch.Tensor, scale: float, need_weights: bool):
        raise NotImplementedError

    @property
    def max_batch_size(self) -> int:
        return self.params.max_batch_size

    @property
    def n_query_groups(self) -> int:
        return self.params.n_query_groups

    @property
    def head_size(self) -> int:
        return self.params.head_size

    @property
    def dtype(self):
        return self.params.dtype

    @property
    def device(self):
        return self.params.device

    @property
    def buffers_are_allocated(self) -> bool:
        raise NotImplementedError

    def allocate(self, device, dtype) -> None:
        raise NotImplementedError

    def deallocate(self) -> None:
        raise NotImplementedError

    def prefill(self, key: torch.Tensor, value: torch.Tensor) -> None:
        raise NotImplementedError

    def write(self, slots: torch.Tensor, key: torch.Tensor, value: torch.Tensor, token_pos: torch.Tensor, input_pos: int) -> None:
        """Write ``key, value (B,G,n,D)`` at ``slots (B,G,n)`` and set
        ``token_pos[b,g,slots] = input_pos + arange(n)``."""
        raise NotImplementedError

    def get_keys_values(self) -> KeysAndValues:
        raise NotImplementedError

    def get_slots(self, slots: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Gather ``(B,G,n,D)`` rows of K and V at ``slots (B,G,n)``."""
        k, v = self.get_keys_values().both()
        idx = slots.to(torch.int64).unsqueeze(-1).expand(-1, -1, -1, self.head_size)
        return k.gather(2, idx), v.gather(2, idx)

    def reset(self) -> None:
        self.current_length = 0
        self.batch_size = None

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        raise NotImplementedError

    def grow(self, new_length: int) -> None:
        if new_length > self.cache_length:
            raise ValueError(f"new length {new_length} exceeds cache_length {self.cache_length}")
        self.current_length = new_length


class DefaultKVCacheBuffers(KVCacheBuffers):
    """Plain buffers in the compute dtype."""

    def __init__(self, params: KVCacheBuffersParams, cache_length: int):
        super().__init__(params, cache_length)
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None

    @property
    def buffers_are_allocated(self) -> bool:
        return self.k is not None

    def allocate(self, device, dtype) -> None:
        if self.k is None or self.k.device != torch.device(device) or self.k.dtype != dtype:
            p = self.params
            shape = (p.max_batch_size, p.n_query_groups, self.cache_length, p.head_size)
            with torch.inference_mode(False):  # persistent state: usable in training passes after a generation
                self.k = torch.zeros(shape, device=device, dtype=dtype)
                self.v = torch.zeros(shape, device=device, dtype=dtype)
            self.params = KVCacheBuffersParams(p.max_batch_size, p.n_query_groups, p.head_size, dtype, torch.device(device))

    def deallocate(self) -> None:
        self.k = self.v = None

    def prefill(self, key, value) -> None:
        B, _, n, _ = key.shape
        self.allocate(key.device, self.params.dtype or key.dtype)
        self.k[:B, :, :n] = key
        self.v[:B, :, :n] = value
        self.batch_size = B
        self.current_length = n

    def write(self, slots, key, value, token_pos, input_pos) -> None:
        ops.cache_write(self.k, self.v, token_pos, slots, key, value, input_pos)

    def get_keys_values(self) -> KeysAndValues:
        B, L = self.batch_size, self.current_length
        return DefaultKeysAndValues(self.k[:B, :, :L], self.v[:B, :, :L])

    def supports_direct_decode(self) -> bool:
        return self.k is not None and self.k.is_cuda and self.k.dtype == torch.bfloat16 and self.head_size == 128

    def decode_attention(self, query, scale, need_weights, **variant):
        """``variant``: ``softcap``, ``sliding_window``, ``token_pos``, ``query_pos`` of :func:`ops.cuda.decode_attention`."""
        from keys_values_b200.ops import cuda as _cu

        return _cu.decode_attention(query, self.k, self.v, scale, self.current_length, need_weights, **variant)

    def size_estimate(self):
        p = self.params
        sz = 2 * p.max_batch_size * p.n_query_groups * self.cache_length * p.head_size * bits_for_torch_dtype(p.dtype or torch.float32)
        return sz, {"buffers": sz}

    @staticmethod
    def size_estimate_apriori(params: KVCacheParams, **kwargs):
        dtype = params.dtype or kwargs.get("dtype") or torch.float32
        sz = 2 * params.max_batch_size * params.n_query_groups * params.cache_length * params.head_size * bits_for_torch_dtype(dtype)
        return sz, {"buffers": sz}
