"""Watch tensors for NaNs and runaway magnitudes while a computation runs.

``track(x, "where")`` returns ``x`` unchanged; once a tracker file is set
(:func:`initialize_weights_tracker`) the first tensor with a NaN, or with an entry above the
threshold, is written to that file and an ``AssertionError`` names the place. On a GPU the check is
one fused reduction (``isnan | abs > thr`` → ``any``) and one scalar read per call, so it is meant
for bisecting a faulty step, not for production runs. Parity: ``keys_values/tools/tracker.py:19-104``.
"""
from __future__ import annotations

from typing import Optional

import torch


class WeightsTracker:
    def __init__(self) -> None:
        self.file_name: Optional[str] = None
        self.threshold: Optional[float] = None
        self.message_postfix: Optional[str] = None

    def initialize(self, file_name: Optional[str], threshold: Optional[float] = None) -> None:
        self.file_name, self.threshold, self.message_postfix = file_name, threshold, None

    def _fail(self, x: torch.Tensor, what: str, msg: Optional[str]) -> None:
        torch.save(x.cpu(), self.file_name)
        parts = [f"Tensor: {what}"] + [m for m in (msg, self.message_postfix) if m]
        raise AssertionError(": ".join(parts))

    def __call__(self, x: torch.Tensor, msg: Optional[str] = None) -> torch.Tensor:
        if self.file_name is None:
            return x
        xd = x.detach()
        nan = torch.isnan(xd)
        big = None if self.threshold is None else xd.abs() > self.threshold
        bad = nan if big is None else nan | big
        if bool(bad.any()):  # the only host read in the common (clean) case
            n_nan = int(nan.sum())
            if n_nan:
                self._fail(xd, f"{n_nan} of {xd.numel()} entries are NaN", msg)
            self._fail(xd, f"No NaNs, but {int(big.sum())} of {xd.numel()} entries are |elem| > {self.threshold}", msg)
        return x


WEIGHTS_TRACKER = WeightsTracker()


def initialize_weights_tracker(file_name: Optional[str], threshold: Optional[float] = None) -> None:
    """Arms the global tracker (``file_name=None`` disarms it)."""
    WEIGHTS_TRACKER.initialize(file_name, threshold)


def track(x: torch.Tensor, msg: Optional[str] = None) -> torch.Tensor:
    return WEIGHTS_TRACKER(x, msg)


def set_message_postfix(postfix: Optional[str]) -> None:
    WEIGHTS_TRACKER.message_postfix = postfix


def track_weights(module: torch.nn.Module, msg: Optional[str] = None) -> None:
    for name, param in module.named_parameters():
        track(param.data, name if msg is None else f"{name}: {msg}")
