"""AdapterV2 (``keys_values/adapter_v2.py``): every linear layer gets a learnable per-output
scale and bias, ``y = scale · (W x + bias)``; only those are trained."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn as nn

from keys_values_b200.config import Config as BaseConfig
from keys_values_b200.models import model as base


@dataclass
class Config(BaseConfig):
    pass


class AdapterV2Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, **kwargs) -> None:
        super().__init__()
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        self.adapter_bias = nn.Parameter(torch.zeros(out_features), requires_grad=False)
        self.adapter_scale = nn.Parameter(torch.ones(out_features), requires_grad=False)

    @property
    def weight(self):
        return self.linear.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.adapter_scale * (self.linear(x) + self.adapter_bias)


def _wrap_linears(module: nn.Module) -> None:
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear):
            w = AdapterV2Linear(child.in_features, child.out_features, bias=child.bias is not None)
            w.linear = child
            setattr(module, name, w)
        else:
            _wrap_linears(child)


class GPT(base.GPT):
    def __init__(self, config: BaseConfig, **mha_kwargs) -> None:
        super().__init__(config, **mha_kwargs)
        _wrap_linears(self)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


def adapter_filter(key: str, value: Any) -> bool:
    return any(s in key for s in ("adapter_bias", "adapter_scale", "adapter_wte", "gating_factor", "norm_", "ln_f"))


def mark_only_adapter_v2_as_trainable(model: nn.Module) -> None:
    for name, p in model.named_parameters():
        p.requires_grad = adapter_filter(name, p)
