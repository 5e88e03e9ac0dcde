"""Mask and matmul helpers of attention (``keys_values/attention/attention_utils.py:36-551``).
The GPU path does not need them (the kernels mask on token positions themselves); they serve
the PyTorch restatement, tests and users who build custom policies."""
from __future__ import annotations

from typing import Optional

import torch

from keys_values_b200.ops.reference import build_mask, sdpa

ENTRIES_PER_GB = 2**28
DEFAULT_TMP_ARRAY_LIMIT_GB = 3


def mask_slice_bool(input_pos: int, num: int, token_positions: torch.Tensor, n_head: int, sliding_window_size: Optional[int] = None) -> torch.Tensor:
    """Boolean mask ``(B, n_head, num, kv)``: True where attention is NOT allowed."""
    B, G, kv = token_positions.shape
    allowed = build_mask(token_positions, input_pos, num, kv, B, G, token_positions.device, sliding_window_size)
    return ~allowed.repeat_interleave(n_head // G, dim=1)


def build_mask_slice(input_pos: int, num: int, token_positions: torch.Tensor, n_head: int, dtype: torch.dtype, sliding_window_size=None) -> torch.Tensor:
    m = mask_slice_bool(input_pos, num, token_positions, n_head, sliding_window_size)
    return torch.zeros(m.shape, dtype=dtype, device=m.device).masked_fill(m, torch.finfo(dtype).min)


def sdpa_attention_weights(query, key, value, scale_factor: float, input_pos: int, token_positions=None, sliding_window_size=None, softcap=None):
    """Attention outputs and summed weights ``(B, G, kv)`` by the plain restatement."""
    return sdpa(query, key, value, scale_factor, input_pos, token_positions, True, sliding_window_size, softcap)


def sample_token_positions(batch_size: int, n_query_groups: int, q_len: int, kv_len: int, input_pos: int, device=None) -> torch.Tensor:
    """Random token positions of an evicted cache that still holds the ``q_len`` newest tokens."""
    out = torch.empty((batch_size, n_query_groups, kv_len), dtype=torch.int32, device=device)
    new = torch.arange(input_pos, input_pos + q_len, device=device)
    for b in range(batch_size):
        for g in range(n_query_groups):
            old = torch.randperm(input_pos, device=device)[: kv_len - q_len]
            allp = torch.cat((old, new))
            out[b, g] = allp[torch.randperm(kv_len, device=device)].to(torch.int32)
    return out
