"""Stand-in for ``litgpt.model``: rotary tables, RMSNorm and the MLP classes."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def build_rope_cache(
    seq_len: int,
    n_elem: int,
    device: Optional[torch.device] = None,
    base: int = 10000,
    condense_ratio: int = 1,
    extra_config: Optional[dict] = None,
    rope_local_base_freq: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables of shape ``(seq_len, n_elem)``; with ``extra_config`` the inverse
    frequencies are rescaled ("factor" alone: all of them; with "original_max_seq_len",
    "low_freq_factor" and "high_freq_factor": smoothly between scaled and unscaled)."""

    def inv_freq(b):
        return 1.0 / (b ** (torch.arange(0, n_elem, 2, device=device).float() / n_elem))

    theta = inv_freq(base)
    if extra_config is not None:
        factor = extra_config["factor"]
        if "original_max_seq_len" in extra_config:
            orig = extra_config["original_max_seq_len"]
            low, high = extra_config["low_freq_factor"], extra_config["high_freq_factor"]
            wavelen = 2 * torch.pi / theta
            smooth = torch.clamp((orig / wavelen - low) / (high - low), min=0.0, max=1.0)
            theta = (1 - smooth) * (theta / factor) + smooth * theta
        else:
            theta = theta / factor
    seq_idx = torch.arange(seq_len, device=device).float() / condense_ratio
    idx_theta = torch.outer(seq_idx, theta).repeat(1, 2)
    if idx_theta.shape[-1] > n_elem > 1:
        idx_theta = idx_theta[..., :n_elem]
    if rope_local_base_freq is not None:
        local = torch.outer(seq_idx, inv_freq(rope_local_base_freq)).repeat(1, 2)
        if local.shape[-1] > n_elem > 1:
            local = local[..., :n_elem]
        idx_theta = torch.stack((idx_theta, local), dim=-1)
    return torch.cos(idx_theta), torch.sin(idx_theta)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates the two halves of the last axis of ``x``; ``cos``/``sin`` are ``(1|B, T, n_elem)``."""
    if cos.dim() != 3:
        raise ValueError(f"cos must be three-dimensional, but shape is {cos.shape}")
    if cos.shape != sin.shape:
        raise ValueError(f"cos, sin must have same shape, but cos.shape={cos.shape}, sin.shape={sin.shape}")
    half = x.size(-1) // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    diff = x.dim() - cos.dim()
    if diff > 0:
        shape = cos.shape[0:1] + (1,) * diff + cos.shape[1:]
        cos, sin = cos.view(*shape), sin.view(*shape)
    return ((x * cos) + (rotated * sin)).to(dtype=x.dtype)


class RMSNorm(nn.Module):
    """Root-mean-square norm computed in fp32."""

    def __init__(self, size: int, dim: int = -1, eps: float = 1e-6, add_unit_offset: bool = False) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size))
        self.eps = eps
        self.dim = dim
        self.add_unit_offset = add_unit_offset

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dtype = x.dtype
        x = x.float()
        norm_x = torch.mean(x * x, dim=self.dim, keepdim=True)
        x_normed = x * torch.rsqrt(norm_x + self.eps)
        weight = (1 + self.weight) if self.add_unit_offset else self.weight
        return (x_normed * weight.float()).to(dtype=dtype)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


class GptNeoxMLP(nn.Module):
    def __init__(self, config, intermediate_size: Optional[int] = None) -> None:
        super().__init__()
        self.intermediate_size = intermediate_size or config.intermediate_size
        self.fc = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.proj = nn.Linear(self.intermediate_size, config.n_embd, bias=config.bias)
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.gelu(self.fc(x), approximate=self.config.gelu_approximate))


class LLaMAMLP(nn.Module):
    def __init__(self, config, intermediate_size: Optional[int] = None) -> None:
        super().__init__()
        self.intermediate_size = intermediate_size or config.intermediate_size
        self.fc_1 = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.fc_2 = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.proj = nn.Linear(self.intermediate_size, config.n_embd, bias=config.bias)
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.silu(self.fc_1(x)) * self.fc_2(x))


class GemmaMLP(LLaMAMLP):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.gelu(self.fc_1(x), approximate=self.config.gelu_approximate) * self.fc_2(x))


class LLaMAMoE(nn.Module):
    def __init__(self, config) -> None:
        super().__init__()
        self.gate = nn.Linear(config.n_embd, config.n_expert, bias=False)
        self.experts = nn.ModuleList(
            LLaMAMLP(config, intermediate_size=config.moe_intermediate_size) for _ in range(config.n_expert)
        )
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.size()
        x = x.view(-1, C)
        router = self.gate(x)
        probs, indices = torch.topk(router, self.config.n_expert_per_token)
        probs = probs.softmax(dim=1, dtype=torch.float).to(dtype=x.dtype)
        masks = (indices.unsqueeze(-1) == torch.arange(self.config.n_expert, device=x.device)).permute(2, 0, 1)
        y = torch.zeros_like(x)
        for mask, expert in zip(masks, self.experts):
            token_idx, expert_idx = torch.where(mask)
            y[token_idx] += probs[token_idx, expert_idx, None] * expert(x[token_idx])
        return y.view(B, T, C)
