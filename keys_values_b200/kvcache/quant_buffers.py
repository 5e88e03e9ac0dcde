"""Quantized KV-cache buffers.

The quantized tensors are the storage format of every layer. One full-precision
scratch pair (:class:`DequantizedKVCacheBuffers`) is *shared by all layers*; a
layer that needs its keys and values claims the scratch, which de-quantizes that
layer's storage into it. Parity: ``keys_values/kvcache/quant_buffers.py:33-947``.

Difference from the reference: new rows are quantized *when they are written*
(one fused kernel writes the full-precision row into the scratch and its
quantized form into storage), because the set of dirty rows is known exactly.
The reference instead tracks dirty slot ranges and quantizes them when the
scratch changes owner. The values seen by attention are the same in both
schemes: rows written since the scratch was claimed are read in full precision,
all older rows have been through ``dq(q(x))``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from keys_values_b200 import ops
from keys_values_b200.attention.base import DefaultKeysAndValues, KeysAndValues
from keys_values_b200.kvcache.base import KVCacheParams, bits_for_torch_dtype
from keys_values_b200.kvcache.buffers import KVCacheBuffers, KVCacheBuffersParams
from keys_values_b200.kvcache.quantize import Quantizer, TorchBasicQuantizer


class DequantizedKVCacheBuffers:
    """Full-precision scratch shared by the quantized buffers of all layers."""

    def __init__(self, params: KVCacheBuffersParams, cache_length: int, max_num_ranges: Optional[int] = None):
        self.params = params
        self.cache_length = cache_length
        self.max_num_ranges = max_num_ranges  # accepted for compatibility; dirty rows are exact here
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.owner: Optional["QuantizedKVCacheBuffers"] = None
        self.num_dequantizations = 0

    def allocate(self, device, dtype) -> None:
        p = self.params
        if self.k is None or self.k.device != torch.device(device) or self.k.dtype != dtype:
            shape = (p.max_batch_size, p.n_query_groups, self.cache_length, p.head_size)
            with torch.inference_mode(False):  # persistent state: usable in training passes after a generation
                self.k = torch.empty(shape, device=device, dtype=dtype)
                self.v = torch.empty(shape, device=device, dtype=dtype)
            self.owner = None

    def deallocate(self) -> None:
        self.k = self.v = None
        self.owner = None

    def claim(self, new_owner: "QuantizedKVCacheBuffers", dequantize: bool = True) -> None:
        if self.owner is new_owner and self.k is not None:
            return
        dtype = self.params.dtype or new_owner.quantizer_k.source_dtype
        self.allocate(new_owner.device, dtype)
        self.owner = new_owner
        if dequantize and new_owner.current_length > 0:
            B, L = new_owner.batch_size, new_owner.current_length
            new_owner.quantizer_k.dequantize(0, L, out=self.k[:B, :, :L])
            new_owner.quantizer_v.dequantize(0, L, out=self.v[:B, :, :L])
            self.num_dequantizations += 1

    def release(self, owner: Optional["QuantizedKVCacheBuffers"] = None) -> None:
        if owner is None or self.owner is owner:
            self.owner = None

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        p = self.params
        sz = 2 * p.max_batch_size * p.n_query_groups * self.cache_length * p.head_size * bits_for_torch_dtype(p.dtype or torch.float32)
        return sz, {"dequant_buffers": sz}


class DequantizedBufferKeysAndValues(DefaultKeysAndValues):
    pass


class QuantizedKVCacheBuffers(KVCacheBuffers):
    def __init__(
        self,
        quantizer_k: Quantizer,
        quantizer_v: Quantizer,
        dequant_buffers: DequantizedKVCacheBuffers,
        debug_label: Optional[str] = None,
    ):
        B, G, C, D = quantizer_k.shape
        params = KVCacheBuffersParams(B, G, D, quantizer_k.source_dtype, quantizer_k.device)
        super().__init__(params, C)
        if quantizer_v.shape != quantizer_k.shape:
            raise ValueError("quantizer_k and quantizer_v must have the same shape")
        self.quantizer_k = quantizer_k
        self.quantizer_v = quantizer_v
        self.dequant_buffers = dequant_buffers
        self.debug_label = debug_label
        self._device = quantizer_k.device
        # Called with ``self`` before the storage of this layer is touched (the
        # offloader uses it to bring the storage onto the device).
        self.before_access: Optional[Callable[["QuantizedKVCacheBuffers"], None]] = None

    @property
    def device(self):
        return self._device

    @property
    def num_bits(self) -> int:
        return self.quantizer_k.num_bits

    @property
    def buffers_are_allocated(self) -> bool:
        return self.quantizer_k.buffers_are_allocated

    def allocate(self, device, dtype=None) -> None:
        self._device = torch.device(device)
        self.quantizer_k.allocate_buffers(device)
        self.quantizer_v.allocate_buffers(device)

    def deallocate(self) -> None:
        self.quantizer_k.deallocate()
        self.quantizer_v.deallocate()
        self.dequant_buffers.release(self)

    def reset(self) -> None:
        super().reset()
        self.dequant_buffers.release(self)

    def _fusable(self) -> bool:
        qk = self.quantizer_k
        return isinstance(qk, TorchBasicQuantizer) and not qk.blocks_over_heads

    def _touch(self) -> None:
        if self.before_access is not None:
            self.before_access(self)

    def prefill(self, key, value) -> None:
        B, _, n, _ = key.shape
        self.allocate(key.device)
        self._touch()
        self.batch_size, self.current_length = B, n
        self.quantizer_k.batch_size = self.quantizer_v.batch_size = B
        self.quantizer_k.quantize(0, n, key)
        self.quantizer_v.quantize(0, n, value)
        # The prefill rows are read back in full precision until the scratch changes owner
        self.dequant_buffers.claim(self, dequantize=False)
        self.dequant_buffers.k[:B, :, :n] = key
        self.dequant_buffers.v[:B, :, :n] = value

    def supports_direct_decode(self) -> bool:
        qk = self.quantizer_k
        # the decode kernel copies cache rows and scale vectors in 16-byte units
        return (self._fusable() and qk.buffers_are_allocated and qk.quant_buffer.is_cuda and self.head_size == 128
                and self.cache_length % 4 == 0)

    def decode_attention(self, query, scale, need_weights, **variant):
        """Attention of one new token straight from the quantized storage; the row
        written by the preceding :meth:`write` is taken in full precision."""
        from keys_values_b200.ops import cuda as _cu

        qk, qv = self.quantizer_k, self.quantizer_v
        slots, key, value = self._last_new
        new_kv = (key[:, :, 0], value[:, :, 0], slots[:, :, 0])
        return _cu.decode_attention(
            query, qk.quant_buffer, qv.quant_buffer, scale, self.current_length, need_weights,
            quant=(qk.quant_scales, qk.quant_zero_points, qv.quant_scales, qv.quant_zero_points, self.num_bits), new_kv=new_kv,
            **variant,
        )

    def write(self, slots, key, value, token_pos, input_pos) -> None:
        self._touch()
        if self.decode_mode:
            # storage only: the full-precision scratch is neither claimed nor filled
            qk, qv = self.quantizer_k, self.quantizer_v
            self.dequant_buffers.release(self)
            ops.cache_write_quant(
                None, None, token_pos, slots, key, value, input_pos,
                qk.quant_buffer, qk.quant_scales, qk.quant_zero_points,
                qv.quant_buffer, qv.quant_scales, qv.quant_zero_points, self.num_bits,
            )
            self._last_new = (slots, key, value)
            return
        self.dequant_buffers.claim(self)
        dq = self.dequant_buffers
        if self._fusable():
            qk, qv = self.quantizer_k, self.quantizer_v
            ops.cache_write_quant(
                dq.k, dq.v, token_pos, slots, key, value, input_pos,
                qk.quant_buffer, qk.quant_scales, qk.quant_zero_points,
                qv.quant_buffer, qv.quant_scales, qv.quant_zero_points, self.num_bits,
            )
        else:
            ops.cache_write(dq.k, dq.v, token_pos, slots, key, value, input_pos)
            self.quantizer_k.quantize_slots(slots, key)
            self.quantizer_v.quantize_slots(slots, value)

    def get_keys_values(self) -> KeysAndValues:
        if self.decode_mode:
            return None
        self._touch()
        self.dequant_buffers.claim(self)
        B, L = self.batch_size, self.current_length
        return DequantizedBufferKeysAndValues(self.dequant_buffers.k[:B, :, :L], self.dequant_buffers.v[:B, :, :L])

    def write_back(self) -> None:
        """Storage is always current (rows are quantized when written)."""

    def drop_association(self) -> None:
        self.dequant_buffers.release(self)

    def quantization_error(self, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        return self.quantizer_k.quantization_error(key) + self.quantizer_v.quantization_error(value)

    def snapshot(self) -> Dict[str, torch.Tensor]:
        """Copy of the quantized storage of the occupied slots (used as KV checkpoint)."""
        self._touch()
        B, L = self.batch_size, self.current_length
        out = {}
        for name, qz in (("k", self.quantizer_k), ("v", self.quantizer_v)):
            out[name + "_q"] = qz.quant_buffer[:B, :, :L].clone()
            if qz.blocks_over_heads:
                out[name + "_s"] = qz.quant_scales[:B, :L].clone()
                out[name + "_z"] = qz.quant_zero_points[:B, :L].clone()
            else:
                out[name + "_s"] = qz.quant_scales[:B, :, :L].clone()
                out[name + "_z"] = qz.quant_zero_points[:B, :, :L].clone()
        return out

    def size_estimate(self):
        sk, _ = self.quantizer_k.size_estimate()
        sv, _ = self.quantizer_v.size_estimate()
        return sk + sv, {"quant_k": sk, "quant_v": sv}

    @staticmethod
    def size_estimate_apriori(params: KVCacheParams, num_bits: int = 8, **kwargs):
        shape = (params.max_batch_size, params.n_query_groups, params.cache_length, params.head_size)
        s, _ = TorchBasicQuantizer.size_estimate_apriori(shape, num_bits, **kwargs)
        return 2 * s, {"quant_k": s, "quant_v": s}


def get_quant_kwargs(params: KVCacheParams, qname: str, cache_kwargs: Dict[str, Any]):
    """Split ``cache_kwargs`` into quantizer arguments and the rest; choose the
    quantizer class for buffer name ``qname`` (``torch-quantized8`` …)."""
    cache_kwargs = dict(cache_kwargs)
    blocks_over_heads = cache_kwargs.pop("blocks_over_heads", False)
    cache_kwargs.pop("tmp_array_limit_gb", None)
    quant_kwargs = dict(
        shape=(params.max_batch_size, params.n_query_groups, params.cache_length, params.head_size),
        source_dtype=params.dtype,
        blocks_over_heads=blocks_over_heads,
    )
    if qname.startswith("torch-quantized"):
        quantizer_type = TorchBasicQuantizer
    elif qname.startswith("bnb-quantized"):
        # The bitsandbytes block-wise quantizer of the reference (keys_values/kvcache/quantize/bitsandbytes.py)
        # is an optional back-end that needs that package; the framework's own storage formats are torch-quantized*.
        raise ImportError(
            f"buffer type {qname!r} needs the optional 'bitsandbytes' package, which this framework does not bind; "
            f"use 'torch-quantized{qname[-1]}' (same bit width, asymmetric per-row quantization) instead"
        )
    else:
        raise ValueError(f"qname = {qname} not supported")
    quant_kwargs["num_bits"] = int(qname[-1])
    return quant_kwargs, quantizer_type, cache_kwargs


def create_quantized_kv_buffers(
    qname: str,
    cache_lengths: List[int],
    cache_params: KVCacheParams,
    cache_kwargs: Optional[Dict[str, Any]] = None,
    dequant_kwargs: Optional[Dict[str, Any]] = None,
    allocate_buffers: bool = False,
    device=None,
    first_block_idx: int = 0,
) -> List[QuantizedKVCacheBuffers]:
    """Quantized buffers for a list of layers; layers with equal cache length
    share one de-quantization scratch."""
    from dataclasses import replace

    cache_kwargs = dict(cache_kwargs or {})
    dequant_kwargs = dict(dequant_kwargs or {})
    scratch: Dict[int, DequantizedKVCacheBuffers] = {}
    result = []
    for i, c_len in enumerate(cache_lengths):
        params = replace(cache_params, cache_length=c_len)
        if c_len not in scratch:
            scratch[c_len] = DequantizedKVCacheBuffers(
                KVCacheBuffersParams.from_params(params, device), c_len, **dequant_kwargs
            )
        quant_kwargs, quantizer_type, _ = get_quant_kwargs(params, qname, cache_kwargs)
        quant_kwargs.update(allocate_buffers=allocate_buffers, device=device)
        result.append(
            QuantizedKVCacheBuffers(
                quantizer_k=quantizer_type(**quant_kwargs),
                quantizer_v=quantizer_type(**quant_kwargs),
                dequant_buffers=scratch[c_len],
                debug_label=f"block{first_block_idx + i}",
            )
        )
    return result
