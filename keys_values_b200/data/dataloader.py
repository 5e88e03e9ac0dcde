"""DataLoader whose batch sampler state can be saved and restored
(``keys_values/data/dataloader.py:56-92``)."""
from __future__ import annotations

from typing import Any, Dict

from torch.utils.data import DataLoader


class MyDataLoader(DataLoader):
    def state_dict(self) -> Dict[str, Any]:
        bs = self.batch_sampler
        return bs.state_dict() if hasattr(bs, "state_dict") else {}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        if hasattr(self.batch_sampler, "load_state_dict") and state:
            self.batch_sampler.load_state_dict(state)


class CycleIterator:
    """Iterates over a loader forever and counts epochs (role of ``litgpt.utils.CycleIterator``)."""

    def __init__(self, iterable):
        self.iterable = iterable
        self.epoch = 0
        self._iterator = None

    def __next__(self):
        if self._iterator is None:
            self._iterator = iter(self.iterable)
        try:
            return next(self._iterator)
        except StopIteration:
            self._iterator = iter(self.iterable)
            self.epoch += 1
            return next(self._iterator)

    def __iter__(self):
        return self
