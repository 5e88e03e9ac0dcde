"""Q-Hitter caches: H2O scores combined with the quantization error of each slot.

``score = c·mm(h2o) + ((c−1)/2)·mm(q_err) + (1−c)``, ``mm`` = min-max normalisation
per batch row, ``q_err = ‖k − dq(q(k))‖ + ‖v − dq(q(v))‖``. Only meaningful with
quantized buffers. Parity: ``keys_values/kvcache/qh2o.py:30-310``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from keys_values_b200.kvcache.h2o import H2OKVCache, VLengthInstantScoreMixin
from keys_values_b200.kvcache.quant_buffers import QuantizedKVCacheBuffers

DEFAULT_COMBINATION_CONSTANT = 0.5


def min_max_normalize(scores: torch.Tensor) -> torch.Tensor:
    flat = scores.reshape(scores.size(0), -1)
    mn = flat.min(dim=-1, keepdim=True)[0]
    denom = flat.max(dim=-1, keepdim=True)[0] - mn
    return ((flat - mn) / denom).view(*scores.shape)


class QuantizedH2OKVCache(H2OKVCache):
    def __init__(self, config, buffers, block_idx, combination_constant: float = DEFAULT_COMBINATION_CONSTANT, scratch_blocksize: Optional[int] = None, **base_kwargs):
        if not isinstance(buffers, QuantizedKVCacheBuffers):
            raise ValueError("qh2o caches can only be used with quantized buffers")
        if not (0 < combination_constant <= 1):
            raise ValueError(f"combination_constant = {combination_constant}, must be in (0, 1]")
        super().__init__(config, buffers, block_idx, **base_kwargs)
        self.combination_constant = combination_constant

    def _score_buffer_names(self) -> List[str]:
        return super()._score_buffer_names() + ["q_errors"]

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 2

    def _initial_scores_in_forward(self, key, value) -> Dict[str, torch.Tensor]:
        d = super()._initial_scores_in_forward(key, value)
        d["q_errors"] = self.kv_buffers.quantization_error(key, value)
        return d

    def _initial_scores_in_prefill(self, key, value) -> Dict[str, torch.Tensor]:
        d = super()._initial_scores_in_prefill(key, value)
        d["q_errors"] = self.kv_buffers.quantization_error(key, value)
        return d

    def _modify_scores(self, scores: torch.Tensor) -> torch.Tensor:
        limit = scores.shape[2]
        c = self.combination_constant
        q_err = self._scores["q_errors"][: self.batch_size, :, :limit]
        return c * min_max_normalize(scores) + ((c - 1) / 2) * min_max_normalize(q_err) + (1 - c)


class QuantizedVLengthH2OKVCache(VLengthInstantScoreMixin, QuantizedH2OKVCache):
    def _score_buffer_names(self) -> List[str]:
        return ["scores", "q_errors", "v_norm"]

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 3
