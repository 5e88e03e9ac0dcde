"""Flat-vector access to the weights or gradients of a module
(``keys_values/optimize/module_wrapper.py:69-251``): one contiguous vector per dtype, with the
layout (name, offset, shape) recorded, so that whole shards move between host and device with
one copy each."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


class AccessWeightsGradients:
    def __init__(self, module: torch.nn.Module, only_trainable: bool = False):
        self.module = module
        self.layout: Dict[torch.dtype, List[Tuple[str, int, torch.Size]]] = {}
        self.sizes: Dict[torch.dtype, int] = {}
        for name, p in module.named_parameters():
            if only_trainable and not p.requires_grad:
                continue
            off = self.sizes.get(p.dtype, 0)
            self.layout.setdefault(p.dtype, []).append((name, off, p.shape))
            self.sizes[p.dtype] = off + p.numel()
        self._params = dict(module.named_parameters())

    def get_weights(self, device=None, pin_memory: bool = False) -> Dict[torch.dtype, torch.Tensor]:
        out = {}
        for dt, entries in self.layout.items():
            dev = device if device is not None else self._params[entries[0][0]].device
            flat = torch.empty(self.sizes[dt], dtype=dt, device=dev, pin_memory=pin_memory and torch.device(dev).type == "cpu" and torch.cuda.is_available())
            for name, off, shape in entries:
                flat[off : off + shape.numel()].copy_(self._params[name].data.reshape(-1), non_blocking=True)
            out[dt] = flat
        return out

    def set_weights(self, flats: Dict[torch.dtype, torch.Tensor]) -> None:
        for dt, entries in self.layout.items():
            for name, off, shape in entries:
                self._params[name].data.copy_(flats[dt][off : off + shape.numel()].view(shape), non_blocking=True)

    def get_gradients(self, device=None) -> Dict[torch.dtype, torch.Tensor]:
        out = {}
        for dt, entries in self.layout.items():
            dev = device if device is not None else self._params[entries[0][0]].device
            flat = torch.zeros(self.sizes[dt], dtype=dt, device=dev)
            for name, off, shape in entries:
                g = self._params[name].grad
                if g is not None:
                    flat[off : off + shape.numel()].copy_(g.reshape(-1), non_blocking=True)
            out[dt] = flat
        return out

    def accumulate_gradients(self, flats: Dict[torch.dtype, torch.Tensor]) -> None:
        """Add flat gradients (possibly on another device) into ``.grad`` of the parameters."""
        for dt, entries in self.layout.items():
            for name, off, shape in entries:
                p = self._params[name]
                g = flats[dt][off : off + shape.numel()].view(shape).to(p.device, non_blocking=True)
                p.grad = g.clone() if p.grad is None else p.grad.add_(g)
