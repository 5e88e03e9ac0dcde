"""Asymmetric affine 8/4-bit row quantizer.

Math (``keys_values/kvcache/quantize/pytorch.py:100-154``): for each block of
values (one ``(b, g, slot)`` row of ``D`` values, or one ``(b, slot)`` row of
``G·D`` values with ``blocks_over_heads``): ``scale = max((max−min)/(2^bits−1),
eps)``, ``zp = −round(min/scale)`` (int32), ``q = clamp(round(x/scale)+zp, 0,
2^bits−1)``, ``x̂ = (q−zp)·scale``; 4-bit storage packs element ``i`` (high nibble)
with element ``i + D/2`` (low nibble). Zero points are kept as int32 in the
state mirror as well (the reference narrows them to uint8 there, which wraps).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from keys_values_b200 import ops
from keys_values_b200.kvcache.quantize.quantization import Quantizer, QuantizerState

MIN_BLOCKSIZE = 16


class TorchBasicQuantizer(Quantizer):
    supported_bits = (4, 8)

    def __init__(self, shape, source_dtype, num_bits: int = 8, blocks_over_heads: bool = False, device=None, allocate_buffers: bool = False, **_):
        super().__init__(shape, source_dtype, num_bits, blocks_over_heads, device)
        if num_bits not in self.supported_bits:
            raise ValueError(f"num_bits = {num_bits}, must be in {self.supported_bits}")
        _, G, _, D = self.shape
        blocksize = G * D if blocks_over_heads else D
        if blocksize < MIN_BLOCKSIZE:
            raise ValueError(f"blocksize = {blocksize} must be at least {MIN_BLOCKSIZE}")
        if num_bits == 4 and D % 2 != 0:
            raise ValueError("head_size must be even for 4-bit quantization")
        self.quant_buffer: Optional[torch.Tensor] = None
        self.quant_scales: Optional[torch.Tensor] = None
        self.quant_zero_points: Optional[torch.Tensor] = None
        if allocate_buffers:
            self.allocate_buffers(device)

    # ------------------------------------------------------------- storage
    @property
    def buffers_are_allocated(self) -> bool:
        return self.quant_buffer is not None

    def _last_dim(self) -> int:
        D = self.shape[-1]
        return D // 2 if self.num_bits == 4 else D

    def allocate_buffers(self, device=None) -> None:
        if device is None:
            device = self._device if self._device is not None else torch.get_default_device()
        device = torch.device(device)
        if self.quant_buffer is not None and self.quant_buffer.device == device:
            return
        B, G, C, _ = self.shape
        self._device = device
        meta_shape = (B, C) if self.blocks_over_heads else (B, G, C)
        with torch.inference_mode(False):  # persistent state: usable in training passes after a generation
            self.quant_buffer = torch.zeros((B, G, C, self._last_dim()), dtype=torch.uint8, device=device)
            self.quant_scales = torch.ones(meta_shape, dtype=torch.float32, device=device)
            self.quant_zero_points = torch.zeros(meta_shape, dtype=torch.int32, device=device)

    def deallocate(self) -> None:
        self.quant_buffer = self.quant_scales = self.quant_zero_points = None

    # ---------------------------------------------------------------- math
    def _quantize_values(self, values: torch.Tensor):
        if not self.blocks_over_heads:
            return ops.quantize_rows(values, self.num_bits)
        B, G, n, D = values.shape
        qmax = float(2**self.num_bits - 1)
        xf = values.float().permute(0, 2, 1, 3).reshape(B, n, G * D)
        mn, mx = xf.amin(-1), xf.amax(-1)
        scale = torch.clamp((mx - mn) / qmax, min=torch.finfo(torch.float32).eps)
        zp = (0 - torch.round(mn / scale)).to(torch.int32)
        q = torch.clamp(torch.round(xf / scale.unsqueeze(-1)) + zp.unsqueeze(-1).float(), 0.0, qmax).to(torch.uint8)
        q = q.view(B, n, G, D).permute(0, 2, 1, 3)
        if self.num_bits == 4:
            half = D // 2
            q = (q[..., :half] << 4) | q[..., half:]
        return q.contiguous(), scale, zp

    def _dequantize_values(self, q, scale, zp, out=None):
        if not self.blocks_over_heads:
            return ops.dequantize_rows(q, scale, zp, self.num_bits, self.source_dtype, out)
        if self.num_bits == 4:
            q = torch.cat(((q >> 4) & 0xF, q & 0xF), dim=-1)
        res = ((q.float() - zp.float()[:, None, :, None]) * scale[:, None, :, None]).to(self.source_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def quantize(self, start: int, end: int, values: torch.Tensor) -> None:
        self.allocate_buffers(values.device)
        B = values.shape[0]
        self.batch_size = B
        q, s, z = self._quantize_values(values)
        self.quant_buffer[:B, :, start:end] = q
        if self.blocks_over_heads:
            self.quant_scales[:B, start:end] = s
            self.quant_zero_points[:B, start:end] = z
        else:
            self.quant_scales[:B, :, start:end] = s
            self.quant_zero_points[:B, :, start:end] = z

    def quantize_slots(self, slots: torch.Tensor, values: torch.Tensor) -> None:
        self.allocate_buffers(values.device)
        B = values.shape[0]
        q, s, z = self._quantize_values(values)
        idx = slots.to(torch.int64)
        self.quant_buffer[:B].scatter_(2, idx.unsqueeze(-1).expand(-1, -1, -1, q.shape[-1]), q)
        if self.blocks_over_heads:
            # slots must then agree across the group axis
            self.quant_scales[:B].scatter_(1, idx[:, 0], s)
            self.quant_zero_points[:B].scatter_(1, idx[:, 0], z)
        else:
            self.quant_scales[:B].scatter_(2, idx, s)
            self.quant_zero_points[:B].scatter_(2, idx, z)

    def dequantize(self, start: int, end: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        B = self.batch_size if self.batch_size is not None else self.max_batch_size
        q = self.quant_buffer[:B, :, start:end]
        if self.blocks_over_heads:
            s, z = self.quant_scales[:B, start:end], self.quant_zero_points[:B, start:end]
        else:
            s, z = self.quant_scales[:B, :, start:end], self.quant_zero_points[:B, :, start:end]
        return self._dequantize_values(q, s, z, out)

    def quantization_error(self, values: torch.Tensor) -> torch.Tensor:
        q, s, z = self._quantize_values(values)
        deq = self._dequantize_values(q, s, z)
        return torch.linalg.vector_norm(values.float() - deq.float(), dim=-1)

    # ---------------------------------------------------------------- misc
    def create_quantizer_state(self, device=None, pin_memory: bool = False) -> "TorchBasicQuantizerState":
        return TorchBasicQuantizerState(self, device, pin_memory)

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        return self.size_estimate_apriori(self.shape, self.num_bits, blocks_over_heads=self.blocks_over_heads)

    @staticmethod
    def size_estimate_apriori(shape, num_bits: int, blocks_over_heads: bool = False, **kwargs):
        B, G, C, D = shape
        sz_buf = B * G * C * D * num_bits
        n_meta = B * C if blocks_over_heads else B * G * C
        sz_meta = n_meta * (32 + 32)
        return sz_buf + sz_meta, {"quant_buffer": sz_buf, "quant_scales_zero_points": sz_meta}


class TorchBasicQuantizerState(QuantizerState):
    def __init__(self, quantizer: TorchBasicQuantizer, device=None, pin_memory: bool = False):
        super().__init__(quantizer, device)
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self._q = self._s = self._z = None

    def _alloc_like(self, t: torch.Tensor) -> torch.Tensor:
        return torch.empty(t.shape, dtype=t.dtype, device=self.device, pin_memory=self.pin_memory and self.device.type == "cpu")

    def copy_(self) -> None:
        qz = self.quantizer
        if not qz.buffers_are_allocated:
            raise RuntimeError("quantizer buffers are not allocated")
        if self._q is None:
            self._q, self._s, self._z = (self._alloc_like(t) for t in (qz.quant_buffer, qz.quant_scales, qz.quant_zero_points))
        self._q.copy_(qz.quant_buffer, non_blocking=True)
        self._s.copy_(qz.quant_scales, non_blocking=True)
        self._z.copy_(qz.quant_zero_points, non_blocking=True)
        self.batch_size = qz.batch_size

    def restore(self) -> None:
        if self._q is None:
            raise RuntimeError("copy_() must be called before restore()")
        qz = self.quantizer
        qz.allocate_buffers(qz.device)
        qz.quant_buffer.copy_(self._q, non_blocking=True)
        qz.quant_scales.copy_(self._s, non_blocking=True)
        qz.quant_zero_points.copy_(self._z, non_blocking=True)
        qz.batch_size = self.batch_size
