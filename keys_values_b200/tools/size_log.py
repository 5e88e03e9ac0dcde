"""Norms of weights and gradients per step (``keys_values/tools/size_log.py:186``) and detection
of unexpected weight changes (``keys_values/tools/tracker.py:19``)."""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, List, Optional

import torch


class SizeWeightsGradientsLog:
    def __init__(self, model: torch.nn.Module, path: Optional[Path] = None, only_trainable: bool = True):
        self.model, self.path, self.only_trainable = model, path, only_trainable
        self.rows: List[Dict[str, float]] = []

    @torch.no_grad()
    def log(self, step: int) -> Dict[str, float]:
        w2 = g2 = 0.0
        gmax = 0.0
        for _, p in self.model.named_parameters():
            if self.only_trainable and not p.requires_grad:
                continue
            w2 += float(p.float().pow(2).sum())
            if p.grad is not None:
                g2 += float(p.grad.float().pow(2).sum())
                gmax = max(gmax, float(p.grad.float().abs().max()))
        row = {"step": step, "weight_norm": w2**0.5, "grad_norm": g2**0.5, "grad_absmax": gmax}
        self.rows.append(row)
        if self.path is not None:
            with open(self.path, "w", newline="") as fp:
                w = csv.DictWriter(fp, fieldnames=list(row.keys()))
                w.writeheader()
                w.writerows(self.rows)
        return row


class WeightsTracker:
    """Remembers checksums of selected weights; ``changed()`` names those that differ now."""

    def __init__(self, model: torch.nn.Module, predicate=None):
        self.model, self.predicate = model, predicate or (lambda n, p: not p.requires_grad)
        self._sums: Dict[str, float] = {}
        self.snapshot()

    @torch.no_grad()
    def snapshot(self) -> None:
        self._sums = {n: float(p.double().sum()) for n, p in self.model.named_parameters() if self.predicate(n, p)}

    @torch.no_grad()
    def changed(self) -> List[str]:
        return [n for n, p in self.model.named_parameters() if n in self._sums and float(p.double().sum()) != self._sums[n]]
