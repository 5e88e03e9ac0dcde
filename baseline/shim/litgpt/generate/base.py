"""Stand-in for ``litgpt.generate.base``: the token sampler."""
from typing import Optional

import torch


def multinomial_num_samples_1(probs: torch.Tensor) -> torch.Tensor:
    return torch.multinomial(probs, num_samples=1)


def sample_top_p(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    sorted_logits, sorted_indices = torch.sort(logits, descending=False)
    cumulative = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
    remove = cumulative <= (1 - top_p)
    remove[-1:] = 0
    return logits.masked_fill(remove.scatter(0, sorted_indices, remove), float("-inf"))


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, top_p: float = 1.0) -> torch.Tensor:
    if top_p < 0.0 or top_p > 1.0:
        raise ValueError(f"top_p must be in [0, 1], got {top_p}")
    logits = logits[0, -1]
    if top_k is not None:
        v, i = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = torch.full_like(logits, float("-inf")).scatter_(-1, i, v)
    if temperature > 0.0 or top_p > 0.0:
        if temperature > 0.0:
            logits = logits / temperature
        if top_p < 1.0:
            logits = sample_top_p(logits, top_p)
        return multinomial_num_samples_1(torch.nn.functional.softmax(logits, dim=-1))
    return torch.argmax(logits, dim=-1, keepdim=True)
