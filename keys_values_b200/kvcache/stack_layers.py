"""A few consecutive blocks as one callable unit (``keys_values/kvcache/stack_layers.py:24-163``):
the unit of a row of cells in the backward pass."""
from __future__ import annotations

from typing import List, Sequence

import torch


class CellBlocks:
    def __init__(self, config):
        self.config = config

    @property
    def first_layer_idx(self) -> int:
        raise NotImplementedError

    @property
    def num_layers(self) -> int:
        raise NotImplementedError

    def blocks(self) -> List[torch.nn.Module]:
        raise NotImplementedError

    def assign_kv_caches(self, caches: Sequence) -> None:
        for b, c in zip(self.blocks(), caches):
            b.attn.kv_cache = c

    def get_kv_caches(self) -> List:
        return [b.attn.kv_cache for b in self.blocks()]

    def forward(self, x: torch.Tensor, idx: torch.Tensor, mha, chunk_sizes=None) -> torch.Tensor:
        for b in self.blocks():
            x = b(x, idx, mha, chunk_sizes=chunk_sizes)
        return x

    __call__ = forward


class DefaultCellBlocks(CellBlocks):
    def __init__(self, model, first_layer_idx: int, num_layers: int):
        super().__init__(model.config)
        if not (0 <= first_layer_idx and first_layer_idx + num_layers <= model.config.n_layer):
            raise ValueError("layer range out of bounds")
        self._model, self._first, self._num = model, first_layer_idx, num_layers

    @property
    def first_layer_idx(self) -> int:
        return self._first

    @property
    def num_layers(self) -> int:
        return self._num

    def blocks(self):
        return list(self._model.transformer.h[self._first : self._first + self._num])
