"""Quantizer interface for KV-cache storage.

A quantizer owns the quantized form of *one* of the two buffers (K or V) of one
layer, shape ``(max_batch, n_query_groups, cache_length, head_size)``, and converts
slot ranges or scattered slots to and from the compute dtype. Parity:
``keys_values/kvcache/quantize/quantization.py:25-358``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch


class Quantizer(torch.nn.Module):
    def __init__(self, shape: Tuple[int, int, int, int], source_dtype: torch.dtype, num_bits: int, blocks_over_heads: bool = False, device=None):
        super().__init__()
        if len(shape) != 4:
            raise ValueError("shape must be (max_batch_size, n_query_groups, cache_length, head_size)")
        self.shape = tuple(shape)
        self.source_dtype = source_dtype
        self.num_bits = num_bits
        self.blocks_over_heads = blocks_over_heads
        self._device = None if device is None else torch.device(device)
        self.batch_size: Optional[int] = None

    @property
    def device(self):
        return self._device

    @property
    def max_batch_size(self) -> int:
        return self.shape[0]

    @property
    def buffers_are_allocated(self) -> bool:
        raise NotImplementedError

    def allocate_buffers(self, device=None) -> None:
        raise NotImplementedError

    def deallocate(self) -> None:
        raise NotImplementedError

    def quantize(self, start: int, end: int, values: torch.Tensor) -> None:
        """Quantize ``values (B,G,end-start,D)`` into slots ``[start, end)``."""
        raise NotImplementedError

    def quantize_slots(self, slots: torch.Tensor, values: torch.Tensor) -> None:
        """Quantize ``values (B,G,n,D)`` into slots ``slots (B,G,n)``."""
        raise NotImplementedError

    def dequantize(self, start: int, end: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """De-quantize slots ``[start, end)`` to ``(B,G,end-start,D)`` in ``source_dtype``."""
        raise NotImplementedError

    def quantization_error(self, values: torch.Tensor) -> torch.Tensor:
        """``‖x − dq(q(x))‖₂`` per row, fp32 ``(B,G,n)`` (used by the Q-Hitter scores)."""
        raise NotImplementedError

    def create_quantizer_state(self, device=None, pin_memory: bool = False) -> "QuantizerState":
        raise NotImplementedError

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        raise NotImplementedError

    @staticmethod
    def size_estimate_apriori(shape, num_bits: int, **kwargs) -> Tuple[int, Dict[str, int]]:
        raise NotImplementedError


class QuantizerState:
    """Mirror of a quantizer's storage on another device (normally pinned host
    memory). ``copy_()`` stores the quantizer's current content, ``restore()``
    writes it back; both are asynchronous on the stream they are called on."""

    def __init__(self, quantizer: Quantizer, device=None):
        self.quantizer = quantizer
        self.device = torch.device("cpu") if device is None else torch.device(device)
        self.batch_size: Optional[int] = None

    def copy_(self) -> None:
        raise NotImplementedError

    def restore(self) -> None:
        raise NotImplementedError
