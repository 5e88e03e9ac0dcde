"""LLaMA-Adapter v1 (``keys_values/adapter.py``): a learnable prefix of ``adapter_prompt_length``
embeddings per layer (from ``adapter_start_layer`` on) attended to with a zero-initialised gate:
``y = attn(x) + g · softmax(q · k_prefix) v_prefix``. Not used by the long-context commands."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from keys_values_b200.config import Config as BaseConfig
from keys_values_b200.models import model as base


@dataclass
class Config(BaseConfig):
    adapter_prompt_length: int = 10
    adapter_start_layer: int = 2


class CausalSelfAttention(base.CausalSelfAttention):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__(config, block_idx, kv_cache)
        if block_idx >= config.adapter_start_layer:
            self.adapter_wte = nn.Embedding(config.adapter_prompt_length, config.n_embd)
            self.gating_factor = nn.Parameter(torch.zeros(1, 1, config.n_head, 1))

    def forward(self, x, token_idx, mha, chunk_sizes=None):
        y = super().forward(x, token_idx, mha, chunk_sizes)
        if self.block_idx < self.config.adapter_start_layer:
            return y
        c = self.config
        B, T, _ = x.shape
        H, G, D = c.n_head, c.n_query_groups, c.head_size
        prefix = self.adapter_wte.weight.unsqueeze(0)
        qkv_p = self.qkv(prefix)
        _, k_p, v_p = qkv_p.split((H * D, G * D, G * D), dim=-1)
        q = self.qkv(x)[..., : H * D].view(B, T, H, D)
        k_p = k_p.view(1, -1, G, D).repeat_interleave(H // G, dim=2)
        v_p = v_p.view(1, -1, G, D).repeat_interleave(H // G, dim=2)
        att = torch.einsum("bthd,xphd->bthp", q, k_p) / math.sqrt(D)
        ay = torch.einsum("bthp,xphd->bthd", att.softmax(-1), v_p)
        return y + self.proj((self.gating_factor * ay).reshape(B, T, H * D))


class Block(base.Block):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__(config, block_idx, kv_cache)
        self.attn = CausalSelfAttention(config, block_idx, kv_cache)


class GPT(base.GPT):
    def _make_block(self, config, block_idx):
        return Block(config, block_idx)


def adapter_filter(key: str, value) -> bool:
    return "adapter_wte" in key or "gating_factor" in key


def mark_only_adapter_as_trainable(model: nn.Module) -> None:
    for name, p in model.named_parameters():
        p.requires_grad = adapter_filter(name, p)
