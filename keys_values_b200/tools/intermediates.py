"""Recording and comparison of intermediate activations (``keys_values/tools/intermediates.py:51``):
register on a model, run two code paths (for example chunked vs whole-sequence forward, or
forward vs the recomputation inside the backward pass) and list where they start to differ."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


class DebugIntermediates:
    def __init__(self, predicate=None):
        self.predicate = predicate or (lambda name: True)
        self.entries: Dict[str, torch.Tensor] = {}
        self._handles: List = []
        self._counter: Dict[str, int] = {}

    def __call__(self, value: torch.Tensor, postfix: str, prefix: str = "") -> None:
        name = prefix + postfix
        k = self._counter.get(name, 0)
        self._counter[name] = k + 1
        self.entries[f"{name}#{k}"] = value.detach().float().cpu().clone()

    def register(self, model: torch.nn.Module) -> None:
        for name, mod in model.named_modules():
            if name and self.predicate(name):
                self._handles.append(mod.register_forward_hook(lambda m, i, o, n=name: self(o if torch.is_tensor(o) else o[0], n) if torch.is_tensor(o) or (isinstance(o, tuple) and torch.is_tensor(o[0])) else None))

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def clear(self) -> None:
        self.entries.clear()
        self._counter.clear()

    @staticmethod
    def compare(a: "DebugIntermediates", b: "DebugIntermediates", atol: float = 1e-5, rtol: float = 1e-4) -> List[Tuple[str, float]]:
        """Entries present in both whose values differ, with the largest absolute difference."""
        out = []
        for k, va in a.entries.items():
            vb = b.entries.get(k)
            if vb is None or va.shape != vb.shape:
                continue
            if not torch.allclose(va, vb, atol=atol, rtol=rtol):
                out.append((k, float((va - vb).abs().max())))
        return out
