"""Host offload of quantized KV-cache storage.

Only the layer that is being processed keeps its quantized storage on the GPU;
all other layers live in pinned host memory. Transfers are ``cudaMemcpyAsync``
on a dedicated side stream, fenced with events: the storage of the next layer is
prefetched while the current layer computes, and the write-back of the previous
layer overlaps as well. Parity: ``keys_values/kvcache/offloading.py:28-156``
(which copies on the current stream, without overlap).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from keys_values_b200.kvcache.quant_buffers import QuantizedKVCacheBuffers


class KVCacheOffloader:
    def __init__(self, buffers: List[QuantizedKVCacheBuffers], pin_memory: bool = True, prefetch: bool = True):
        self.buffers = buffers
        self.pin_memory = pin_memory
        self.prefetch = prefetch
        self.states_k = [None] * len(buffers)
        self.states_v = [None] * len(buffers)
        self.resident: set = set()
        self.active: Optional[int] = None
        self._stream = None
        self._ready = {}  # layer -> event recorded on the side stream after H2D
        self.num_h2d = self.num_d2h = 0
        for i, b in enumerate(buffers):
            b.before_access = self._make_callback(i)

    def _make_callback(self, idx: int):
        def quantizer_callback(buf: QuantizedKVCacheBuffers) -> None:
            self.activate(idx)

        return quantizer_callback

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        return self._stream

    def _ensure_states(self, idx: int) -> None:
        if self.states_k[idx] is None:
            b = self.buffers[idx]
            self.states_k[idx] = b.quantizer_k.create_quantizer_state(device="cpu", pin_memory=self.pin_memory)
            self.states_v[idx] = b.quantizer_v.create_quantizer_state(device="cpu", pin_memory=self.pin_memory)

    def _offload(self, idx: int) -> None:
        """Device → host for layer ``idx`` and release of its device storage."""
        b = self.buffers[idx]
        if not b.buffers_are_allocated:
            self.resident.discard(idx)
            return
        self._ensure_states(idx)
        dev = b.quantizer_k.quant_buffer.device
        side = self._side_stream(dev)
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self.states_k[idx].copy_()
                self.states_v[idx].copy_()
                for qz in (b.quantizer_k, b.quantizer_v):
                    for t in (qz.quant_buffer, qz.quant_scales, qz.quant_zero_points):
                        t.record_stream(side)
        else:
            self.states_k[idx].copy_()
            self.states_v[idx].copy_()
        self.num_d2h += 1
        b.quantizer_k.deallocate()
        b.quantizer_v.deallocate()
        b.dequant_buffers.release(b)
        self.resident.discard(idx)

    def _fetch(self, idx: int, dev) -> None:
        """Host → device for layer ``idx`` (no-op if it has never been offloaded)."""
        if idx in self.resident:
            return
        b = self.buffers[idx]
        if self.states_k[idx] is not None and self.states_k[idx]._q is not None:
            side = self._side_stream(torch.device(dev))
            if side is not None:
                with torch.cuda.stream(side):
                    self.states_k[idx].restore()
                    self.states_v[idx].restore()
                    ev = torch.cuda.Event()
                    ev.record(side)
                self._ready[idx] = ev
            else:
                self.states_k[idx].restore()
                self.states_v[idx].restore()
            self.num_h2d += 1
        self.resident.add(idx)

    def activate(self, idx: int) -> None:
        if self.active == idx and idx in self.resident:
            return
        b = self.buffers[idx]
        dev = b.device if b.device is not None else torch.device("cpu")
        prev = self.active
        self._fetch(idx, dev)
        ev = self._ready.pop(idx, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        self.active = idx
        if prev is not None and prev != idx and prev in self.resident:
            self._offload(prev)
        if self.prefetch and len(self.buffers) > 1:
            nxt = (idx + 1) % len(self.buffers)
            if nxt != idx and self.buffers[nxt].device is not None:
                self._fetch(nxt, self.buffers[nxt].device)

    def flush(self) -> None:
        """Offload every resident layer (end of a forward pass)."""
        for idx in list(self.resident):
            self._offload(idx)
        self.active = None
        if self._stream is not None:
            self._stream.synchronize()

    def reset(self) -> None:
        self.resident.clear()
        self._ready.clear()
        self.active = None
        for s in self.states_k + self.states_v:
            if s is not None:
                s._q = s._s = s._z = None


def quantizer_callback(offloader: KVCacheOffloader, idx: int):
    return offloader._make_callback(idx)
