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


QUANTILES = ("0.5", "0.9", "0.99", "max")


class SizeLogMapper:
    r"""Maps parameter names to the rows of the per-weight tables. ``rules``: ``(regex, label)`` pairs tried in
    order; parameters whose name matches a rule are pooled under ``label`` (with ``{0}``, ``{1}`` … replaced by the
    regex groups, e.g. ``(r"transformer\.h\.(\d+)\.attn\.qkv\.lora_[AB]", "layer {0} qkv LoRA")``); parameters that
    match no rule keep their own name (``keep_unmatched``) or are left out. Role of ``SizeLogMapper`` /
    ``SizeLogMapperRule`` in ``keys_values/tools/size_log.py:44-110``."""

    def __init__(self, rules=(), keep_unmatched: bool = True):
        import re

        self.rules = [(re.compile(rx), label) for rx, label in rules]
        self.keep_unmatched = keep_unmatched
        self.labels: List[str] = []
        self._index: Dict[str, int] = {}

    def index_of(self, name: str) -> Optional[int]:
        label = None
        for rx, lab in self.rules:
            m = rx.search(name)
            if m:
                label = lab.format(*m.groups())
                break
        if label is None:
            if not self.keep_unmatched:
                return None
            label = name
        if label not in self._index:
            self._index[label] = len(self.labels)
            self.labels.append(label)
        return self._index[label]


class PerWeightSizeLog:
    """Per step and per (group of) parameter(s): quantiles 0.5 / 0.9 / 0.99 and the maximum of the absolute values
    of the weights and of their gradients. ``write(dir)`` leaves ``size_weights.csv`` and ``size_gradients.csv``
    (columns ``step, weight_idx, q, value``) and ``weight_names.csv`` (``weight_idx, name``), the tables that
    :mod:`keys_values_b200.tools.plot_size_log` draws (``keys_values/tools/size_log.py:186-366``)."""

    def __init__(self, model: torch.nn.Module, mapper: Optional[SizeLogMapper] = None, only_trainable: bool = True, max_samples: int = 1 << 20):
        self.model, self.mapper, self.only_trainable, self.max_samples = model, mapper or SizeLogMapper(), only_trainable, max_samples
        self.weights: List[Dict] = []
        self.gradients: List[Dict] = []

    def _quantiles(self, parts: List[torch.Tensor]) -> Dict[str, float]:
        x = torch.cat([t.detach().float().abs().reshape(-1) for t in parts])
        mx = float(x.max()) if x.numel() else 0.0
        if x.numel() > self.max_samples:  # quantiles from an evenly spaced sample, the maximum from everything
            x = x[:: x.numel() // self.max_samples + 1]
        qs = torch.quantile(x.cpu(), torch.tensor([0.5, 0.9, 0.99])) if x.numel() else torch.zeros(3)
        return {"0.5": float(qs[0]), "0.9": float(qs[1]), "0.99": float(qs[2]), "max": mx}

    @torch.no_grad()
    def log(self, step: int) -> None:
        groups_w: Dict[int, List[torch.Tensor]] = {}
        groups_g: Dict[int, List[torch.Tensor]] = {}
        for name, p in self.model.named_parameters():
            if self.only_trainable and not p.requires_grad:
                continue
            idx = self.mapper.index_of(name)
            if idx is None:
                continue
            groups_w.setdefault(idx, []).append(p)
            if p.grad is not None:
                groups_g.setdefault(idx, []).append(p.grad)
        for table, groups in ((self.weights, groups_w), (self.gradients, groups_g)):
            for idx, parts in sorted(groups.items()):
                for q, v in self._quantiles(parts).items():
                    table.append({"step": step, "weight_idx": idx, "q": q, "value": v})

    def write(self, out_dir: Path) -> None:
        out_dir = Path(out_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        for fname, table in (("size_weights.csv", self.weights), ("size_gradients.csv", self.gradients)):
            with open(out_dir / fname, "w", newline="") as fp:
                w = csv.DictWriter(fp, fieldnames=["step", "weight_idx", "q", "value"])
                w.writeheader()
                w.writerows(table)
        with open(out_dir / "weight_names.csv", "w", newline="") as fp:
            w = csv.writer(fp)
            w.writerow(["weight_idx", "name"])
            w.writerows(enumerate(self.mapper.labels))


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
