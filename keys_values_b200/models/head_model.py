"""Loss heads that are evaluated chunk by chunk.

A head returns *un-normalised* per-row sums for a chunk; the long-context wrapper
adds the chunks and divides by :meth:`HeadModel.num_target_entries`. Targets are
right-aligned with the model outputs of the chunk. Parity:
``keys_values/head_model.py:24-431``.
"""
from __future__ import annotations

import copy
from typing import List, Optional, Union

import torch
import torch.nn.functional as F

from keys_values_b200 import ops

from keys_values_b200.config import Config

IGNORE_INDEX = -100


class HeadModel(torch.nn.Module):
    NAME = "head"

    def needs_logits(self) -> bool:
        raise NotImplementedError

    def forward(self, model_outputs: torch.Tensor, targets: Optional[torch.Tensor], input_pos: int) -> torch.Tensor:
        raise NotImplementedError

    def num_target_entries(self, targets: torch.Tensor) -> Optional[torch.Tensor]:
        raise NotImplementedError

    @staticmethod
    def _check_model_outputs_targets(model_outputs, targets, final_dim: int) -> Optional[int]:
        if model_outputs.ndim != 3 or model_outputs.shape[-1] != final_dim:
            raise ValueError(f"model_outputs.shape = {tuple(model_outputs.shape)}, must be 3D with final size {final_dim}")
        if targets is None:
            return None
        if targets.ndim != 2 or targets.shape[0] != model_outputs.shape[0]:
            raise ValueError(f"model_outputs.shape = {tuple(model_outputs.shape)}, targets.shape = {tuple(targets.shape)}: Not compatible")
        diff = model_outputs.shape[-2] - targets.shape[-1]
        if diff < 0:
            raise ValueError("model_outputs must not be shorter than targets")
        return diff

    def clone(self, device=None) -> "HeadModel":
        other = copy.deepcopy(self)
        return other if device is None else other.to(device)


class CrossEntropyOnLogits(HeadModel):
    """Next-token cross-entropy; ``targets == -100`` are ignored."""

    NAME = "next_token_prediction"

    def __init__(self, config: Config):
        super().__init__()
        self._vocab_size = config.padded_vocab_size

    def needs_logits(self) -> bool:
        return True

    def forward(self, model_outputs, targets, input_pos):
        if targets is None:
            return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
        diff = self._check_model_outputs_targets(model_outputs, targets, self._vocab_size)
        logits = model_outputs[:, diff:, :]
        losses = ops.cross_entropy_rows(logits.reshape(-1, self._vocab_size), targets, IGNORE_INDEX)
        return losses.view(targets.shape).sum(dim=-1)

    def num_target_entries(self, targets: torch.Tensor) -> Optional[torch.Tensor]:
        return (targets != IGNORE_INDEX).sum(dim=-1)


class SequenceClassificationOnLogits(HeadModel):
    """Class labels are single tokens: cross-entropy over the logits of
    ``class_label_tokens`` at the final position; ``targets (B,1)`` in
    ``[0, num_classes)``."""

    NAME = "seq_classification_on_logits"

    def __init__(self, config: Config, class_label_tokens: List[int]):
        super().__init__()
        self._vocab_size = config.padded_vocab_size
        self.num_classes = len(class_label_tokens)
        if self.num_classes < 2:
            raise ValueError(f"class_label_tokens = {class_label_tokens} must have at least 2 elements")
        if not all(x == int(x) and 0 <= x < self._vocab_size for x in class_label_tokens):
            raise ValueError(f"class_label_tokens = {class_label_tokens} must be in [0, {self._vocab_size})")
        if len(set(class_label_tokens)) != self.num_classes:
            raise ValueError(f"class_label_tokens = {class_label_tokens} must not have duplicates")
        self.class_label_tokens = tuple(class_label_tokens)

    def needs_logits(self) -> bool:
        return True

    def forward(self, model_outputs, targets, input_pos):
        if targets is None:
            return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
        if targets.shape[-1] != 1:
            raise ValueError(f"targets.length = {targets.shape[-1]}, must be 1")
        self._check_model_outputs_targets(model_outputs, targets, self._vocab_size)
        selected = model_outputs[:, -1, list(self.class_label_tokens)].float()
        return F.cross_entropy(selected, targets.reshape(-1), reduction="none")

    def num_target_entries(self, targets):
        return None


SUPPORTED_POOL_TYPES = ("last", "mean")


class SequenceClassification(HeadModel):
    """Linear head on a pooled state (``last`` token or ``mean`` over tokens)."""

    NAME = "seq_classification"

    def __init__(self, config: Config, num_classes: int = 2, pool_type: str = "last"):
        super().__init__()
        if num_classes < 2:
            raise ValueError(f"num_classes = {num_classes} must be >= 2")
        if pool_type not in SUPPORTED_POOL_TYPES:
            raise ValueError(f"pool_type = {pool_type} must be one of {SUPPORTED_POOL_TYPES}")
        self.num_classes, self.n_embd, self.pool_type = num_classes, config.n_embd, pool_type
        self.linear_head = torch.nn.Linear(config.n_embd, num_classes, bias=True)
        self._num_tokens = None
        self._accumulated_state = None

    def needs_logits(self) -> bool:
        return False

    def forward(self, model_outputs, targets, input_pos) -> Union[torch.Tensor, float]:
        self._check_model_outputs_targets(model_outputs, targets, self.n_embd)
        if targets is not None and targets.shape[-1] != 1:
            raise ValueError(f"targets.length = {targets.shape[-1]}, must be 1")
        num = model_outputs.shape[-2]
        if input_pos == 0:
            self._accumulated_state = 0 if self.pool_type == "mean" else None
            self._num_tokens = 0
        else:
            assert self._num_tokens is not None, "First call must be with input_pos=0"
            assert input_pos == self._num_tokens, f"input_pos = {input_pos} != {self._num_tokens} = num_tokens"
        if self.pool_type == "mean":
            self._accumulated_state = model_outputs.sum(dim=-2) + self._accumulated_state
        self._num_tokens += num
        if targets is None:
            return 0
        state = self._accumulated_state / self._num_tokens if self.pool_type == "mean" else model_outputs[..., -1, :]
        self._accumulated_state = None
        logits = self.linear_head(state)
        return F.cross_entropy(logits.float(), targets.reshape(-1), reduction="none")

    def num_target_entries(self, targets):
        return None


class HeadModelFactory:
    """Creates a head by name (``keys_values/head_model_factory.py:34-67``)."""

    SUPPORTED = (CrossEntropyOnLogits.NAME, SequenceClassificationOnLogits.NAME, SequenceClassification.NAME)

    @staticmethod
    def create(name: str, config: Config, **kwargs) -> HeadModel:
        if name == CrossEntropyOnLogits.NAME:
            return CrossEntropyOnLogits(config)
        if name == SequenceClassificationOnLogits.NAME:
            return SequenceClassificationOnLogits(config, **kwargs)
        if name == SequenceClassification.NAME:
            return SequenceClassification(config, **kwargs)
        raise ValueError(f"name = {name} not supported; must be in {HeadModelFactory.SUPPORTED}")

    @staticmethod
    def is_supported(name: str) -> bool:
        return name in HeadModelFactory.SUPPORTED
