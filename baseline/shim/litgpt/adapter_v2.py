"""Stand-in for ``litgpt.adapter_v2``."""
from typing import Any

import torch
import torch.nn as nn


class AdapterV2Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, **kwargs: Any) -> None:
        super().__init__()
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        self.adapter_bias = nn.Parameter(torch.zeros(out_features), requires_grad=False)
        self.adapter_scale = nn.Parameter(torch.ones(out_features), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.adapter_scale * (self.linear(x) + self.adapter_bias)

    def reset_parameters(self) -> None:
        nn.init.zeros_(self.adapter_bias)
        nn.init.ones_(self.adapter_scale)
