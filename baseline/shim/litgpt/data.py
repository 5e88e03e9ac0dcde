"""Stand-in for ``litgpt.data``."""
from __future__ import annotations

from typing import Optional


class DataModule:
    """Base of the reference's data modules (``connect`` / ``setup`` / ``*_dataloader``)."""

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length: Optional[int] = None) -> None:
        pass

    def prepare_data(self) -> None:
        pass

    def setup(self, stage: str = "") -> None:
        pass

    def train_dataloader(self):
        raise NotImplementedError

    def val_dataloader(self):
        raise NotImplementedError


class Alpaca(DataModule):
    pass
