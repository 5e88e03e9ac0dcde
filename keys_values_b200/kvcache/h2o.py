"""Heavy-hitter-oracle (H2O) caches.

``scores (B,G,C)`` fp32 accumulate the attention weights each slot received
(summed over queries, averaged over the query heads of the group); when the cache
is full, the slots with the lowest scores are overwritten next. Parity:
``keys_values/kvcache/h2o.py:28-625``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from keys_values_b200 import ops
from keys_values_b200.kvcache.attn_weights import AttnWeightsKVCache


def _topk_smallest(s: torch.Tensor, k: int) -> torch.Tensor:
    k = min(k, s.shape[-1])
    if k == s.shape[-1]:
        return torch.argsort(s, dim=-1).to(torch.int32)
    return torch.topk(s, k=k, dim=-1, largest=False, sorted=True)[1].to(torch.int32)


class H2OKVCache(AttnWeightsKVCache):
    """Improved H2O: per batch row and KV head decisions; optional normalisation of
    the cumulative score by the age of the token (``normalize_scores``)."""

    def __init__(self, config, buffers, block_idx, normalize_scores: bool = False, **base_kwargs):
        super().__init__(config, buffers, block_idx, **base_kwargs)
        self.normalize_scores = normalize_scores

    def _score_buffer_names(self) -> List[str]:
        return ["scores"]

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 1

    @property
    def scores(self) -> torch.Tensor:
        return self._scores["scores"]

    # -- hooks for subclasses
    def _instantaneous_score(self, attn_weights: torch.Tensor, query_length: int) -> torch.Tensor:
        return attn_weights

    def _modify_scores(self, scores: torch.Tensor) -> Optional[torch.Tensor]:
        """Return transformed selection scores, or ``None`` for "unchanged"."""
        return None

    def _plain(self) -> bool:
        return type(self)._instantaneous_score is H2OKVCache._instantaneous_score and type(self)._modify_scores is H2OKVCache._modify_scores

    # slots selected after a single-token step (the next step of a generation needs one; a longer
    # chunk that follows selects again from the same scores, see ``_reselect``)
    DECODE_SELECT = 8

    def _fused_select(self, attn_weights: Optional[torch.Tensor], k: int) -> torch.Tensor:
        """Fused: scores += w (skipped for ``None``), (age-normalise), k smallest among the evictable
        slots. The result lives in a buffer kept per ``k``, so that a captured decode step and the
        eager steps before it exchange the slots through one address."""
        B = self.batch_size
        key = (B, k)
        out = self._select_out.get(key) if hasattr(self, "_select_out") else None
        if out is None or out.device != self.scores.device:
            if not hasattr(self, "_select_out"):
                self._select_out = {}
            with torch.inference_mode(False):
                out = self._select_out[key] = torch.empty((B, self.n_query_groups, k), dtype=torch.int32, device=self.scores.device)
        return ops.h2o_update(
            self.scores[:B], attn_weights, k, self.cache_length - self.grace_period,
            normalize=self.normalize_scores, token_pos=self.token_pos[:B],
            input_pos=self.input_pos, prefill_length=self.prefill_length, out=out,
        )

    def _reselect(self, num: int) -> torch.Tensor:
        if self._plain() and self.max_chunk_size is not None and self.current_length == self.cache_length:
            return self._fused_select(None, max(num, self.max_chunk_size))
        return super()._reselect(num)

    def _select_after_accumulate(self, attn_weights: torch.Tensor, num: int) -> None:
        B, L, C = self.batch_size, self.current_length, self.cache_length
        limit = C - self.grace_period
        if L == C and self._plain() and self.max_chunk_size is not None:
            k = min(self.max_chunk_size, self.DECODE_SELECT) if num == 1 else self.max_chunk_size
            self._next_positions = self._fused_select(attn_weights, k)
            return
        self.scores[:B, :, :L] += self._instantaneous_score(attn_weights, num)
        if L < C:
            self._next_positions = None
            return
        s = self.scores[:B, :, :limit]
        if self.normalize_scores:
            tp = self.token_pos[:B, :, :limit].clamp(min=self.prefill_length - 1)
            s = s / (self.input_pos - tp).to(torch.float32)
        mod = self._modify_scores(s)
        if mod is not None:
            s = mod
        k = self.max_chunk_size if self.max_chunk_size is not None else limit
        self._next_positions = _topk_smallest(s, k)


class VLengthInstantScoreMixin:
    """Instantaneous score ``n · (w ⊙ ‖v‖) / Σ_slots (w ⊙ ‖v‖)`` with a per-slot
    ``v_norm`` buffer filled at prefill and on every write."""

    def _instantaneous_score(self, attn_weights: torch.Tensor, query_length: int) -> torch.Tensor:
        s = self._scores["v_norm"][: self.batch_size, :, : self.current_length] * attn_weights
        return s / s.sum(dim=-1, keepdim=True) * query_length

    def _initial_scores_in_forward(self, key, value) -> Dict[str, torch.Tensor]:
        d = super()._initial_scores_in_forward(key, value)
        d["v_norm"] = torch.linalg.vector_norm(value.float(), dim=-1)
        return d

    def _initial_scores_in_prefill(self, key, value) -> Dict[str, torch.Tensor]:
        d = super()._initial_scores_in_prefill(key, value)
        d["v_norm"] = torch.linalg.vector_norm(value.float(), dim=-1)
        return d


class VLengthH2OKVCache(VLengthInstantScoreMixin, H2OKVCache):
    def _score_buffer_names(self) -> List[str]:
        return ["scores", "v_norm"]

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 2


class H2OOriginalKVCache(AttnWeightsKVCache):
    """H2O as published (Zhang et al., NeurIPS 2023): scores are summed over the
    batch dimension and one slot choice is shared by all batch rows."""

    def __init__(self, config, buffers, block_idx, **base_kwargs):
        for name in ("normalize_scores",):
            if name in base_kwargs:
                raise ValueError(f"Parameter {name} not supported for this class. Use 'H2OKVCache' instead.")
        super().__init__(config, buffers, block_idx, **base_kwargs)

    def _score_buffer_names(self) -> List[str]:
        return ["scores"]

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 1

    @property
    def scores(self) -> torch.Tensor:
        return self._scores["scores"]

    def _select_after_accumulate(self, attn_weights: torch.Tensor, num: int) -> None:
        B, L, C = self.batch_size, self.current_length, self.cache_length
        self.scores[:B, :, :L] += attn_weights.sum(0, keepdim=True)
        if L < C:
            self._next_positions = None
            return
        limit = C - self.grace_period
        k = self.max_chunk_size if self.max_chunk_size is not None else limit
        self._next_positions = _topk_smallest(self.scores[:B, :, :limit], k)
