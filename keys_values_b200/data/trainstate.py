"""Dataset part of a training state (``keys_values/data/trainstate.py:19-34``)."""
from __future__ import annotations

from typing import Dict

import torch


class DataTrainState:
    """What a dataset must remember so that a resumed run sees the same data: every random choice
    made while loading it that its metadata does not already fix (the position of the batch
    iterator is kept by the sampler, not here)."""

    def state_dict(self) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def load_state_dict(self, state_dict: Dict[str, torch.Tensor]) -> None:
        raise NotImplementedError


class SeedTrainState(DataTrainState):
    """The common case: one seed determines shuffles and sub-sampling."""

    def __init__(self, seed: int = 0):
        self.seed = int(seed)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"seed": torch.tensor(self.seed, dtype=torch.int64)}

    def load_state_dict(self, state_dict: Dict[str, torch.Tensor]) -> None:
        self.seed = int(state_dict["seed"])
