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

    def attend(self, qkv, token_idx, mha, chunk_sizes=None):
        """Attention over the sequence plus, from ``adapter_start_layer`` on, the gated attention of the same
        queries (after QK norm and RoPE) over the learnable prefix: ``y + g_h · softmax(q k_p^T / sqrt(D)) v_p`` per
        head, added BEFORE the output projection (one projection, one bias). The prefix keys and values are the
        K and V parts of ``qkv(prefix)``, without position encoding."""
        c = self.config
        use_prefix = self.block_idx >= c.adapter_start_layer
        if use_prefix:
            input_pos = 0 if self.kv_cache is None else self.kv_cache.input_pos  # before the cache moves on
            q, _, _ = self._split_norm_rope(qkv, mha, input_pos)  # (B, H, T, D)
        y = super().attend(qkv, token_idx, mha, chunk_sizes)
        if not use_prefix:
            return y
        B, T, _ = qkv.shape
        H, G, D = c.n_head, c.n_query_groups, c.head_size
        prefix = self.adapter_wte.weight.unsqueeze(0).to(qkv.dtype)
        _, k_p, v_p = self.qkv(prefix).split((H * D, G * D, G * D), dim=-1)
        k_p = k_p.view(-1, G, D).repeat_interleave(H // G, dim=1)  # (P, H, D)
        v_p = v_p.view(-1, G, D).repeat_interleave(H // G, dim=1)
        att = torch.einsum("bhtd,phd->bhtp", q.float(), k_p.float()) / math.sqrt(D)
        ay = torch.einsum("bhtp,phd->bthd", att.softmax(-1), v_p.float())  # (B, T, H, D)
        return y + (self.gating_factor.float() * ay).reshape(B, T, H * D).to(y.dtype)


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
