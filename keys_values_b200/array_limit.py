"""Mutable limit on the size of temporary arrays with a reduction ladder for
out-of-memory retries (``keys_values/array_limit.py:29-64``). Most temporaries of
this framework are pre-sized, so the ladder rarely matters; it is kept for the
heads that materialise logits and for compatibility."""
from __future__ import annotations

from typing import Optional

REDUCTION_FACTORS = (3 / 4, 1 / 2, 3 / 8, 1 / 4, 3 / 16, 1 / 8, 1 / 16, 1 / 32, 1 / 64)


class TemporaryArrayLimit:
    def __init__(self, init_val: float, name: str = "tmp_array_limit_gb"):
        if init_val <= 0:
            raise ValueError("init_val must be positive")
        self._init_val = float(init_val)
        self.name = name
        self._step = 0

    def __call__(self) -> float:
        if self._step == 0:
            return self._init_val
        return self._init_val * REDUCTION_FACTORS[self._step - 1]

    def can_reduce(self) -> bool:
        return self._step < len(REDUCTION_FACTORS)

    def reduce(self) -> Optional[float]:
        """Next lower limit, or ``None`` if the ladder is exhausted."""
        if not self.can_reduce():
            return None
        self._step += 1
        return self()

    def reset(self) -> None:
        self._step = 0
