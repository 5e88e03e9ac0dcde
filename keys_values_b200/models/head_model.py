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
    def _target_offset(model_outputs: torch.Tensor, targets: Optional[torch.Tensor], width: int) -> Optional[int]:
        """Number of leading positions of the chunk that carry no target: targets are right-aligned with
        the chunk's outputs ``(B, T, width)``. ``None`` without targets. Raises on mismatched shapes."""
        shape = tuple(model_outputs.shape)
        if len(shape) != 3 or shape[2] != width:
            raise ValueError(f"head expects outputs of shape (batch, tokens, {width}), got {shape}")
        if targets is None:
            return None
        if targets.ndim != 2 or targets.shape[0] != shape[0] or targets.shape[1] > shape[1]:
            raise ValueError(f"targets of shape {tuple(targets.shape)} do not fit outputs of shape {shape}: "
                             "same batch size and at most as many positions are required")
        return shape[1] - targets.shape[1]

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
        diff = self._target_offset(model_outputs, targets, self._vocab_size)
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
        labels = tuple(int(t) for t in class_label_tokens)
        problems = []
        if len(labels) < 2:
            problems.append("fewer than two classes")
        if any(a != b for a, b in zip(labels, class_label_tokens)) or any(not 0 <= t < self._vocab_size for t in labels):
            problems.append(f"token ids outside 0..{self._vocab_size - 1}")
        if len(set(labels)) < len(labels):
            problems.append("repeated token ids")
        if problems:
            raise ValueError(f"class_label_tokens {list(class_label_tokens)}: " + ", ".join(problems))
        self.num_classes = len(labels)
        self.class_label_tokens = labels

    def needs_logits(self) -> bool:
        return True

    def forward(self, model_outputs, targets, input_pos):
        if targets is None:
            return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
        if targets.shape[-1] != 1:
            raise ValueError(f"targets.length = {targets.shape[-1]}, must be 1")
        self._target_offset(model_outputs, targets, self._vocab_size)
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
        if num_classes < 2 or pool_type not in SUPPORTED_POOL_TYPES:
            raise ValueError(f"need num_classes >= 2 and pool_type in {SUPPORTED_POOL_TYPES}, got {num_classes} and {pool_type!r}")
        self.num_classes, self.n_embd, self.pool_type = num_classes, config.n_embd, pool_type
        self.linear_head = torch.nn.Linear(config.n_embd, num_classes, bias=True)
        self._seen = 0       # tokens of the current sequence consumed so far
        self._running = None  # sum of their hidden states (mean pooling only)

    def needs_logits(self) -> bool:
        return False

    def forward(self, model_outputs, targets, input_pos) -> Union[torch.Tensor, float]:
        """Consumes the hidden states of one chunk. Chunks of a sequence arrive in order, the first one with
        ``input_pos == 0``; the chunk that carries the ``(B, 1)`` class targets ends the sequence and returns
        the per-row cross-entropy, all earlier chunks return 0."""
        self._target_offset(model_outputs, targets, self.n_embd)
        if targets is not None and targets.shape[1] != 1:
            raise ValueError(f"one class label per row is expected, got targets of shape {tuple(targets.shape)}")
        if input_pos == 0:
            self._seen, self._running = 0, None
        elif input_pos != self._seen:
            raise ValueError(f"chunks must arrive in order: got input_pos {input_pos} after {self._seen} tokens")
        if self.pool_type == "mean":
            chunk_sum = model_outputs.sum(dim=1)
            self._running = chunk_sum if self._running is None else self._running + chunk_sum
        self._seen += model_outputs.shape[1]
        if targets is None:
            return 0
        pooled = self._running / self._seen if self.pool_type == "mean" else model_outputs[:, -1, :]
        self._running = None
        return F.cross_entropy(self.linear_head(pooled).float(), targets.reshape(-1), reduction="none")

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
