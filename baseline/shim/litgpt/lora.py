"""Stand-in for ``litgpt.lora``: the LoRA layer classes the reference derives from."""
from __future__ import annotations

import math
from typing import Any, Dict, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F


class LoRALayer(nn.Module):
    def __init__(self, r: int, lora_alpha: int, lora_dropout: float):
        super().__init__()
        assert r >= 0
        self.r = r
        self.lora_alpha = lora_alpha
        self.lora_dropout = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else (lambda x: x)
        self.merged = False


class LoRALinear(LoRALayer):
    def __init__(self, in_features: int, out_features: int, r: int = 0, lora_alpha: int = 1,
                 lora_dropout: float = 0.0, **kwargs: Any):
        super().__init__(r=r, lora_alpha=lora_alpha, lora_dropout=lora_dropout)
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        if r > 0:
            self.lora_A = nn.Parameter(torch.empty((r, in_features)))
            self.lora_B = nn.Parameter(torch.empty((out_features, r)))
            self.scaling = self.lora_alpha / self.r
            self.reset_parameters()

    def reset_parameters(self) -> None:
        if hasattr(self, "lora_A"):
            nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B)

    def get_lora_AB(self) -> torch.Tensor:
        return (self.lora_B @ self.lora_A) * self.scaling

    def merge(self) -> None:
        if self.r > 0 and not self.merged:
            self.linear.weight.data += self.get_lora_AB().to(self.linear.weight.data.device)
            self.merged = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        pretrained = self.linear(x)
        if self.r == 0 or self.merged:
            return pretrained
        lora = (self.lora_dropout(x) @ self.lora_A.transpose(0, 1) @ self.lora_B.transpose(0, 1)) * self.scaling
        return pretrained + lora


class LoRAQKVLinear(LoRALinear):
    def __init__(self, in_features: int, head_size: int, n_head: int, n_query_groups: int, r: int = 0,
                 lora_alpha: int = 1, lora_dropout: float = 0.0,
                 enable_lora: Union[bool, Tuple[bool, bool, bool]] = False, **kwargs: Any):
        super(LoRALinear, self).__init__(r=r, lora_alpha=lora_alpha, lora_dropout=lora_dropout)
        out_features = head_size * (n_head + 2 * n_query_groups)
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        self.head_size, self.n_head, self.n_query_groups = head_size, n_head, n_query_groups
        if isinstance(enable_lora, bool):
            enable_lora = [enable_lora] * 3
        self.enable_lora = enable_lora
        self._all_qkv_shapes = (head_size * n_head, head_size * n_query_groups, head_size * n_query_groups)
        if r > 0 and any(enable_lora):
            self.lora_A = nn.Parameter(torch.empty((r * sum(enable_lora), in_features)))
            self.qkv_shapes = [s for s, e in zip(self._all_qkv_shapes, enable_lora) if e]
            self.lora_B = nn.Parameter(torch.empty(sum(self.qkv_shapes), r))
            self.scaling = self.lora_alpha / self.r
            self.reset_parameters()

    @property
    def lora_ind(self) -> torch.Tensor:
        if not hasattr(self, "_lora_ind"):
            off, parts = 0, []
            for enable, size in zip(self.enable_lora, self._all_qkv_shapes):
                if enable:
                    parts.append(torch.arange(off, off + size, device=self.linear.weight.device))
                off += size
            self.register_buffer("_lora_ind", torch.cat(parts), persistent=False)
        return self._lora_ind

    def zero_pad(self, x: torch.Tensor) -> torch.Tensor:
        """Scatters the columns of the enabled parts into a zero tensor of the full q|k|v width."""
        if all(self.enable_lora):
            return x
        result = x.new_zeros(*x.shape[:-1], self.linear.out_features)
        return result.index_copy_(dim=-1, index=self.lora_ind.to(x.device), source=x)

    def conv1d(self, input: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """Applies one B matrix per enabled part to its r rows of ``input`` ``(B, r·parts, T)``."""
        if self.n_head == self.n_query_groups:
            return F.conv1d(input, weight, groups=sum(self.enable_lora))
        inputs = input.chunk(sum(self.enable_lora), dim=1)
        weights = weight.split(self.qkv_shapes)
        return torch.cat([F.conv1d(a, b) for a, b in zip(inputs, weights)], dim=1)

    def get_lora_AB(self) -> torch.Tensor:
        lora = self.conv1d(self.lora_A.data.unsqueeze(0), self.lora_B.data.unsqueeze(-1)).squeeze(0)
        return self.zero_pad(lora.T * self.scaling).T

    def merge(self) -> None:
        if self.r > 0 and any(self.enable_lora) and not self.merged:
            super().merge()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        pretrained = self.linear(x)
        if self.r == 0 or not any(self.enable_lora) or self.merged:
            return pretrained
        after_A = F.linear(self.lora_dropout(x), self.lora_A)
        after_B = self.conv1d(after_A.transpose(-2, -1), self.lora_B.unsqueeze(-1)).transpose(-2, -1)
        return pretrained + self.zero_pad(after_B) * self.scaling


def create_lora_linear(config, in_size: int, out_size: int, bias=None, use_r=None) -> LoRALinear:
    if bias is None:
        bias = config.bias
    if use_r is None:
        use_r = config.lora_mlp
    return LoRALinear(in_size, out_size, bias=bias, r=(config.lora_r if use_r else 0),
                      lora_alpha=config.lora_alpha, lora_dropout=config.lora_dropout)


def mark_only_lora_as_trainable(model: nn.Module, bias: str = "none") -> None:
    for n, p in model.named_parameters():
        if "lora_" not in n:
            p.requires_grad = False
    if bias == "none":
        return
    if bias == "all":
        for n, p in model.named_parameters():
            if "bias" in n:
                p.requires_grad = True
    elif bias == "lora_only":
        for m in model.modules():
            if isinstance(m, LoRALayer) and hasattr(m, "bias") and m.bias is not None:
                m.bias.requires_grad = True
    else:
        raise NotImplementedError


def lora_filter(key: str, value: Any) -> bool:
    return "lora_" in key


def merge_lora_weights(model: nn.Module) -> None:
    for module in model.modules():
        if isinstance(module, LoRALinear):
            module.merge()
