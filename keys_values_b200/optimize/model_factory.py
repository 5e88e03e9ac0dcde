"""GPU copies of parts of a host-resident model (weight-offload mode)
(``keys_values/optimize/model_factory.py:38-818``, ``clone_model.py:33-141``).

Shard names: ``wte`` (embedding), ``lm_head`` (final norm + head) and ``h{a}:{b}`` (blocks
``a..b-1``). A shard is materialised on the device from the flat weight vectors of the host
model, used for one row of the backward pass, and its gradients go back as flat vectors."""
from __future__ import annotations

import copy
import re
from typing import List, Tuple

import torch

from keys_values_b200.optimize.module_wrapper import AccessWeightsGradients


def names_and_modules_for_shard(gpt_model, shard: str) -> List[Tuple[str, torch.nn.Module]]:
    if shard == "wte":
        return [("transformer.wte", gpt_model.transformer.wte)]
    if shard == "lm_head":
        return [("transformer.ln_f", gpt_model.transformer.ln_f), ("lm_head", gpt_model.lm_head)]
    m = re.fullmatch(r"h(\d+):(\d+)", shard)
    if not m:
        raise ValueError(f"shard = {shard}: must be 'wte', 'lm_head' or 'h<a>:<b>'")
    a, b = int(m.group(1)), int(m.group(2))
    if not (0 <= a < b <= gpt_model.config.n_layer):
        raise ValueError(f"shard = {shard} out of range for {gpt_model.config.n_layer} layers")
    return [(f"transformer.h.{i}", gpt_model.transformer.h[i]) for i in range(a, b)]


def clone_model_shard_via_flat_vectors(gpt_model, shard: str, device) -> List[Tuple[str, torch.nn.Module]]:
    """Deep copies of the modules of ``shard`` on ``device`` (caches are not copied); weights
    travel as one flat vector per dtype and module."""
    out = []
    for name, mod in names_and_modules_for_shard(gpt_model, shard):
        caches = []
        for sub in mod.modules():
            if hasattr(sub, "kv_cache"):
                caches.append((sub, sub.kv_cache))
                sub.kv_cache = None
        try:
            acc = AccessWeightsGradients(mod)
            flats = {dt: f.to(device, non_blocking=True) for dt, f in acc.get_weights(pin_memory=True).items()}
            clone = copy.deepcopy(mod).to(device)
            AccessWeightsGradients(clone).set_weights(flats)
        finally:
            for sub, c in caches:
                sub.kv_cache = c
        out.append((name, clone))
    return out


class ModelFromFlatVectorsFactory:
    """Creates device shards of a host model and returns their gradients to it."""

    def __init__(self, gpt_model, device):
        self.gpt_model, self.device = gpt_model, torch.device(device)

    def create(self, shard: str) -> List[Tuple[str, torch.nn.Module]]:
        return clone_model_shard_via_flat_vectors(self.gpt_model, shard, self.device)

    def return_gradients(self, shard: str, clones: List[Tuple[str, torch.nn.Module]]) -> None:
        for (name, host_mod), (_, dev_mod) in zip(names_and_modules_for_shard(self.gpt_model, shard), clones):
            grads = AccessWeightsGradients(dev_mod).get_gradients()
            AccessWeightsGradients(host_mod).accumulate_gradients(grads)


class GPTShardCellBlock:
    """Device copies of the blocks of shard ``h{a}:{b}`` as one callable unit with the interface of
    :class:`keys_values_b200.kvcache.stack_layers.CellBlocks` (``keys_values/optimize/model_factory.py:444-489``)."""

    def __init__(self, gpt_model, shard: str, device):
        m = re.fullmatch(r"h(\d+):(\d+)", shard)
        if not m:
            raise ValueError("shard must be a stack of layers 'h<a>:<b>'")
        self.config = gpt_model.config
        self._first = int(m.group(1))
        self._factory = ModelFromFlatVectorsFactory(gpt_model, device)
        self._shard = shard
        self._clones = self._factory.create(shard)

    @property
    def first_layer_idx(self) -> int:
        return self._first

    @property
    def num_layers(self) -> int:
        return len(self._clones)

    def blocks(self) -> List[torch.nn.Module]:
        return [mod for _, mod in self._clones]

    def assign_kv_caches(self, caches) -> None:
        for b, c in zip(self.blocks(), caches):
            b.attn.kv_cache = c

    def get_kv_caches(self) -> List:
        return [b.attn.kv_cache for b in self.blocks()]

    def forward(self, x: torch.Tensor, idx: torch.Tensor, mha, chunk_sizes=None) -> torch.Tensor:
        for b in self.blocks():
            x = b(x, idx, mha, chunk_sizes=chunk_sizes)
        return x

    __call__ = forward

    def return_gradients(self) -> None:
        """Accumulate the gradients of the copies into the host model."""
        self._factory.return_gradients(self._shard, self._clones)
