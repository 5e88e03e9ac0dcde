"""Checkpoint stores used between the forward and the backward pass.

* :class:`LayerInputCheckpoints`: inputs of the first layer of every row (and
  the final hidden states) for the whole sequence, ``(B, T, E)`` each, written
  cell by cell during the forward pass.
* :class:`KVCheckpoints`: snapshot of every layer's cache (quantized storage if
  the cache is quantized) at every cell boundary.

Both live in device memory by default; with ``offload=True`` they are moved to
(pinned) host memory by asynchronous copies on a side stream and brought back on
demand. Layer inputs can additionally be stored in int8/int4 (``qname``). Parity:
``keys_values/kvcache/gradient/checkpoints.py:28-1013``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from keys_values_b200 import ops


def _bits_from_qname(qname: Optional[str]) -> Optional[int]:
    if qname is None or qname == "default":
        return None
    if qname.endswith("quantized8"):
        return 8
    if qname.endswith("quantized4"):
        return 4
    raise ValueError(f"qname = {qname} not supported for checkpoints")


class _SideStream:
    """Lazily created copy stream per device."""

    _streams: Dict[int, Any] = {}

    @classmethod
    def get(cls, device: torch.device):
        if device.type != "cuda":
            return None
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._streams:
            cls._streams[idx] = torch.cuda.Stream(device=device)
        return cls._streams[idx]


def to_host_async(t: torch.Tensor, pin_memory: bool) -> Tuple[torch.Tensor, Any]:
    """Copy ``t`` to host memory on the side stream; returns ``(host_tensor, event)``."""
    if t.device.type != "cuda":
        return t.clone(), None
    side = _SideStream.get(t.device)
    if pin_memory:
        from keys_values_b200.utils.host_pool import pinned_empty

        host = pinned_empty(t.shape, t.dtype)  # a range of the pinned pool: no cudaHostAlloc per checkpoint
    else:
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu")
    side.wait_stream(torch.cuda.current_stream(t.device))
    with torch.cuda.stream(side):
        host.copy_(t, non_blocking=True)
        t.record_stream(side)
        ev = torch.cuda.Event()
        ev.record(side)
    return host, ev


def to_device_async(host: torch.Tensor, device: torch.device, event=None) -> torch.Tensor:
    """Copy a host tensor back; the current stream waits for the transfer."""
    if device.type != "cuda":
        return host
    side = _SideStream.get(device)
    if event is not None:
        side.wait_event(event)
    with torch.cuda.stream(side):
        out = host.to(device, non_blocking=True)
        done = torch.cuda.Event()
        done.record(side)
    torch.cuda.current_stream(device).wait_event(done)
    out.record_stream(torch.cuda.current_stream(device))
    return out


class LayerInputCheckpoints:
    def __init__(
        self,
        layer_indices: List[int],
        batch_size: int,
        seq_length: int,
        n_embd: int,
        dtype: torch.dtype,
        device,
        offload: bool = False,
        pin_memory: bool = True,
        qname: Optional[str] = None,
    ):
        self.slots = {l: i for i, l in enumerate(layer_indices)}
        self.dtype = dtype
        self.device = torch.device(device)
        self.offload = offload and self.device.type == "cuda"
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self.bits = _bits_from_qname(qname)
        self.shape = (batch_size, seq_length, n_embd)
        self._dense: Dict[int, torch.Tensor] = {}
        self._pieces: Dict[Tuple[int, int, int], Any] = {}
        if not self.offload and self.bits is None:
            for l in layer_indices:
                self._dense[l] = torch.empty(self.shape, dtype=dtype, device=self.device)

    def write(self, layer_idx: int, start: int, end: int, x: torch.Tensor) -> None:
        if layer_idx in self._dense:
            self._dense[layer_idx][:, start:end] = x
            return
        if self.bits is not None:
            payload = ops.quantize_rows(x.contiguous(), self.bits)
        else:
            payload = (x.contiguous(),)
        if self.offload:
            payload = tuple(to_host_async(t, self.pin_memory) for t in payload)
        self._pieces[(layer_idx, start, end)] = payload

    def read(self, layer_idx: int, start: int, end: int) -> torch.Tensor:
        if layer_idx in self._dense:
            return self._dense[layer_idx][:, start:end]
        payload = self._pieces[(layer_idx, start, end)]
        if self.offload:
            payload = tuple(to_device_async(h, self.device, ev) for h, ev in payload)
        if self.bits is not None:
            q, s, z = payload
            return ops.dequantize_rows(q, s, z, self.bits, self.dtype)
        return payload[0]

    def size_bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self._dense.values())
        for payload in self._pieces.values():
            for t in payload:
                t = t[0] if isinstance(t, tuple) else t
                total += t.numel() * t.element_size()
        return total


class KVCheckpoints:
    """``(layer, cell) → cache snapshot`` as produced by ``kv_snapshot()``."""

    def __init__(self, offload: bool = False, pin_memory: bool = True):
        self.offload = offload
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self._store: Dict[Tuple[int, int], Dict[str, Any]] = {}

    def _map(self, snap: Dict[str, Any], fn) -> Dict[str, Any]:
        out = {}
        for k, v in snap.items():
            if isinstance(v, dict):
                out[k] = self._map(v, fn)
            elif torch.is_tensor(v):
                out[k] = fn(v)
            else:
                out[k] = v
        return out

    def put(self, layer_idx: int, cell_idx: int, snap: Dict[str, Any]) -> None:
        if self.offload:
            dev = snap["token_pos"].device
            snap = self._map(snap, lambda t: to_host_async(t, self.pin_memory))
            snap["_device"] = dev
        self._store[(layer_idx, cell_idx)] = snap

    def get(self, layer_idx: int, cell_idx: int) -> Dict[str, Any]:
        snap = self._store[(layer_idx, cell_idx)]
        if self.offload:
            dev = snap["_device"]

            def back(pair):
                return to_device_async(pair[0], dev, pair[1])

            out = {}
            for k, v in snap.items():
                if k == "_device":
                    continue
                if isinstance(v, dict):
                    out[k] = {kk: back(vv) for kk, vv in v.items()}
                elif isinstance(v, tuple) and torch.is_tensor(v[0]):
                    out[k] = back(v)
                else:
                    out[k] = v
            return out
        return snap
