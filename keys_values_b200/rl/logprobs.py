"""Per-token log-probabilities of long sequences through the chunked forward
(``keys_values/rl/logprobs.py:49-224``). The head collects ``log p(target_t)`` chunk by
chunk instead of summing a loss, so policies with bounded KV caches can score sequences
that do not fit a dense cache."""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F

from keys_values_b200.config import Config
from keys_values_b200.long_context import LongContextInferenceModel
from keys_values_b200.models.head_model import IGNORE_INDEX, HeadModel


class LogProbsHeadModel(HeadModel):
    NAME = "logprobs"

    def __init__(self, config: Config, temperature: float = 1.0):
        super().__init__()
        self._vocab_size = config.padded_vocab_size
        self.temperature = temperature
        self.parts: List[torch.Tensor] = []

    def needs_logits(self) -> bool:
        return True

    def forward(self, model_outputs, targets, input_pos):
        if targets is None:
            return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
        diff = self._target_offset(model_outputs, targets, self._vocab_size)
        logits = model_outputs[:, diff:, :].float() / self.temperature
        safe = targets.clamp(min=0)
        lp = torch.gather(F.log_softmax(logits, dim=-1), 2, safe.unsqueeze(-1)).squeeze(-1)
        lp = lp.masked_fill(targets == IGNORE_INDEX, 0.0)
        self.parts.append(lp)
        return -lp.sum(dim=-1)

    def num_target_entries(self, targets):
        return (targets != IGNORE_INDEX).sum(dim=-1)

    def reset(self) -> None:
        self.parts = []

    def collected(self) -> torch.Tensor:
        return torch.cat(self.parts, dim=1)


@torch.no_grad()
def compute_logprobs(gpt_model, input_ids: torch.Tensor, targets: torch.Tensor, chunk_size: int, temperature: float = 1.0) -> torch.Tensor:
    """``log p(targets)`` per position ``(B, num_targets)``; ``targets`` are right-aligned with
    ``input_ids`` (``-100`` entries give 0)."""
    head = LogProbsHeadModel(gpt_model.config, temperature)
    lcm = LongContextInferenceModel(gpt_model, head, chunk_size=chunk_size)
    lcm(input_ids, targets)
    return head.collected()
