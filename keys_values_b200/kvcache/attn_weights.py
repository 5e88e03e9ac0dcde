"""Base class of score-based eviction caches.

State machine (``keys_values/kvcache/attn_weights.py:325-1029``):

1. ``prefill`` with ``T <= C`` tokens fills slots ``0..T-1``; no attention weights
   are available, so if ``T == C`` the first eviction uses the *initial rule*:
   overwrite slots starting at ``int(keep_initial_fraction · C)``.
2. ``forward`` with ``n`` new tokens writes them at the slots chosen by the last
   update (or free slots while the cache is filling), runs SDPA with weights,
3. ``_update`` accumulates scores and selects the slots to overwrite next:
   the ``max_chunk_size`` lowest scores, or a full ascending sort.

With ``grace_period = g > 0`` the last ``g`` slots are a ring of the most recent
tokens; a token is moved out of the ring (with its score) into an evictable
slot before a new one takes its place, and only slots ``[0, C-g)`` compete.
Slot selection runs on the device; no value is read back to the host.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from keys_values_b200.attention.base import KeysAndValues
from keys_values_b200.kvcache.base import KVCacheParams, KVCacheReplayLog
from keys_values_b200.kvcache.basics import KVCacheWithBuffers

DEFAULT_KEEP_INITIAL_FRACTION = 0.05
DEFAULT_REPLAY_LOG_BLOCKSIZE = 1024


class AttnWeightsReplayLog(KVCacheReplayLog):
    pass


def update_token_positions(token_positions: torch.Tensor, input_pos: int, num: int, batch_size: int, index: Optional[torch.Tensor],
                           grace_period: int = 0, next_grace_pos: Optional[int] = None):
    """Plain-PyTorch statement of what a cache write does to ``token_positions (bs,G,C)`` when ``num``
    tokens from position ``input_pos`` arrive (the CUDA path writes the positions inside the cache-write
    kernel). While the cache fills, slot = position. Once it is full the tokens go to the slots
    ``index (batch_size,G,num)``; with a grace ring in the last ``grace_period`` slots, the
    ``min(num, grace_period)`` oldest ring entries (positions from ``input_pos - grace_period``) move
    to the first slots of ``index`` and the newest tokens take their place in the ring. Returns
    ``None`` or ``(ring_slots (batch_size,G,n2), n1, prefix)`` for the grace case
    (``keys_values/kvcache/attn_weights.py:214-317``)."""
    bs, G, C = token_positions.shape
    if not (1 <= batch_size <= bs and num >= 1 and input_pos >= 0):
        raise ValueError("need 1 <= batch_size <= token_positions.shape[0], num >= 1, input_pos >= 0")
    dev, dt = token_positions.device, token_positions.dtype
    if input_pos < C:
        if input_pos + num > C:
            raise ValueError(f"input_pos + num = {input_pos + num} > cache_length {C} while the cache is filling")
        token_positions[:batch_size, :, input_pos : input_pos + num] = torch.arange(input_pos, input_pos + num, dtype=dt, device=dev)
        return None
    if index is None or tuple(index.shape) != (batch_size, G, num):
        raise ValueError(f"index must have shape {(batch_size, G, num)}")
    result = None
    start = input_pos
    if grace_period > 0:
        if next_grace_pos is None:
            raise ValueError("next_grace_pos is needed with a grace period")
        n2 = min(num, grace_period)
        n1, prefix = num - n2, C - grace_period
        ring = (torch.arange(n2, device=dev) + (next_grace_pos - prefix)) % grace_period + prefix
        token_positions[:batch_size, :, ring] = torch.arange(input_pos + n1, input_pos + num, dtype=dt, device=dev)
        start = input_pos - grace_period
        result = (ring.view(1, 1, n2).expand(batch_size, G, n2), n1, prefix)
    new = torch.arange(start, start + num, dtype=dt, device=dev).view(1, 1, num).expand(batch_size, G, num)
    token_positions[:batch_size].scatter_(-1, index.to(torch.int64), new)
    return result


class AttnWeightsKVCache(KVCacheWithBuffers):
    def __init__(
        self,
        config,
        buffers,
        block_idx: int,
        grace_period: int = 0,
        replay_log_blocksize: Optional[int] = None,
        detach_attn_weights: bool = False,
        keep_initial_fraction: Optional[float] = None,
        max_chunk_size: Optional[int] = None,
        **base_kwargs,
    ):
        super().__init__(config, buffers, block_idx, **base_kwargs)
        C = buffers.cache_length
        if not (0 <= grace_period < C):
            raise ValueError(f"Must have 0 <= grace_period < {C}, but grace_period = {grace_period}")
        if keep_initial_fraction is None:
            keep_initial_fraction = DEFAULT_KEEP_INITIAL_FRACTION
        elif not (0 <= keep_initial_fraction < 1):
            raise ValueError(f"keep_initial_fraction = {keep_initial_fraction}, must be in [0, 1)")
        if max_chunk_size is not None:
            if not (0 < max_chunk_size <= C):
                raise ValueError(f"max_chunk_size = {max_chunk_size}, must be in (0, {C}]")
            if max_chunk_size > C // 2:
                max_chunk_size = None  # no saving over a full sort
        self.grace_period = grace_period
        self.replay_log_blocksize = replay_log_blocksize or DEFAULT_REPLAY_LOG_BLOCKSIZE
        self._keep_initial_fraction = keep_initial_fraction
        self.max_chunk_size = max_chunk_size
        self._next_positions: Optional[torch.Tensor] = None
        self._use_initial_rule: Optional[bool] = None
        self.next_grace_pos: Optional[int] = None
        self.prefill_length: Optional[int] = None
        self._scores: Dict[str, torch.Tensor] = {}
        self.debug_next_positions: Optional[List[torch.Tensor]] = None

    # ------------------------------------------------------------ properties
    def needs_attn_weights(self) -> bool:
        return True

    def update_requires_attn_weights(self) -> bool:
        return True

    def max_forward_length(self) -> int:
        diff = self.cache_length - self.current_length
        result = self.cache_length - self.grace_period
        if diff > 0:
            result = min(result, diff)
        if self.max_chunk_size is not None:
            result = min(result, self.max_chunk_size)
        return result

    def _score_buffer_names(self) -> List[str]:
        return []

    def _score_buffers(self) -> List[Tuple[torch.Tensor, str]]:
        return [(self._scores[name], name) for name in self._score_buffer_names()]

    def _alloc_scores(self, device) -> None:
        shape = (self.max_batch_size, self.n_query_groups, self.cache_length)
        for name in self._score_buffer_names():
            t = self._scores.get(name)
            if t is None or t.device != torch.device(device):
                with torch.inference_mode(False):
                    self._scores[name] = torch.zeros(shape, dtype=torch.float32, device=device)
            else:
                t.zero_()

    def next_positions(self, num: int) -> Optional[torch.Tensor]:
        if self._next_positions is None:
            return None
        if num > self._next_positions.shape[-1]:
            # a single-token step selected only a few slots: select again from the unchanged scores
            self._next_positions = self._reselect(num)
        return self._next_positions[:, :, :num]

    def _reselect(self, num: int) -> torch.Tensor:
        raise IndexError(f"only {self._next_positions.shape[-1]} next positions are available, {num} needed")

    def reset(self) -> None:
        super().reset()
        self._next_positions = None
        self._use_initial_rule = None
        self.next_grace_pos = None
        self.prefill_length = None

    # ------------------------------------------------------------- prefill
    def _initial_scores_in_prefill(self, key, value) -> Dict[str, torch.Tensor]:
        return {}

    def _initial_scores_in_forward(self, key, value) -> Dict[str, torch.Tensor]:
        return {}

    def _prefill(self, key, value, token_idx) -> None:
        super()._prefill(key, value, token_idx)
        B, _, n, _ = key.shape
        self._alloc_scores(key.device)
        for name, vals in self._initial_scores_in_prefill(key, value).items():
            self._scores[name][:B, :, :n] = vals
        self.prefill_length = n
        self._use_initial_rule = n == self.cache_length
        self._next_positions = None
        self.next_grace_pos = self.cache_length - self.grace_period

    # ------------------------------------------------------------- forward
    def _free_slots(self, n: int, B: int, device) -> torch.Tensor:
        L = self.current_length
        return torch.arange(L, L + n, dtype=torch.int32, device=device).view(1, 1, n).expand(B, self.n_query_groups, n)

    def _forward(self, key, value, token_idx) -> KeysAndValues:
        if self._use_initial_rule is None:
            raise IndexError("Cache needs to be initialized with 'prefill' before being used")
        B, _, n, _ = key.shape
        C, g, L = self.cache_length, self.grace_period, self.current_length
        device = key.device
        if L < C:
            if n > C - L:
                raise ValueError(f"key.shape[2] = {n}, must be <= {C - L} as long as the cache is not full")
            index = self._free_slots(n, B, device)
            full = False
        else:
            full = True
            if self._use_initial_rule:
                keep = min(int(self._keep_initial_fraction * C), C - g - n)
                index = torch.arange(keep, keep + n, dtype=torch.int32, device=device).view(1, 1, n).expand(B, self.n_query_groups, n)
                self._use_initial_rule = False
            else:
                index = self.next_positions(n)
                if index is None:
                    raise IndexError("next positions are not set: forward must follow an update")
        if self.debug_next_positions is not None:
            self.debug_next_positions.append(index.detach().clone().cpu())
        init_vals = self._initial_scores_in_forward(key, value)
        if full and g > 0:
            self._forward_grace(index, key, value, init_vals)
        else:
            self.kv_buffers.write(index, key, value, self.token_pos, self.input_pos)
            idx64 = index.to(torch.int64)
            for scores, name in self._score_buffers():
                vals = init_vals.get(name)
                if vals is None:
                    scores[:B].scatter_(2, idx64, 0.0)
                else:
                    scores[:B].scatter_(2, idx64, vals)
        if not full:
            self.kv_buffers.grow(L + n)
        self._log(n, index)
        self._next_positions = None
        return self.kv_buffers.get_keys_values()

    def _forward_grace(self, index, key, value, init_vals) -> None:
        """Full cache with a grace ring: the ``n2 = min(n, g)`` oldest ring entries
        move to ``index[:n2]`` together with their scores and token positions; the
        first ``n1 = n - n2`` new tokens go to ``index[n2:]``, the last ``n2`` new
        tokens take the freed ring slots."""
        B, _, n, D = key.shape
        C, g = self.cache_length, self.grace_period
        prefix = C - g
        n2 = min(n, g)
        n1 = n - n2
        ring = ((torch.arange(n2, device=key.device) + (self.next_grace_pos - prefix)) % g + prefix).to(torch.int32)
        ring = ring.view(1, 1, n2).expand(B, self.n_query_groups, n2)
        k_old, v_old = self.kv_buffers.get_slots(ring)
        ring64 = ring.to(torch.int64)
        oldest_pos = self.input_pos - g
        self.kv_buffers.write(index[:, :, :n2], k_old, v_old, self.token_pos, oldest_pos)
        new_slots = torch.cat((index[:, :, n2:], ring), dim=-1)
        self.kv_buffers.write(new_slots, key, value, self.token_pos, self.input_pos)
        idx64 = index.to(torch.int64)
        for scores, name in self._score_buffers():
            moved = scores[:B].gather(2, ring64)
            vals = init_vals.get(name)
            scores[:B].scatter_(2, idx64[:, :, :n2], moved)
            new_vals = torch.zeros((B, self.n_query_groups, n), dtype=scores.dtype, device=scores.device) if vals is None else vals
            scores[:B].scatter_(2, new_slots.to(torch.int64), new_vals)
        if n1 == 0:
            self.next_grace_pos = (self.next_grace_pos - prefix + n) % g + prefix

    # -------------------------------------------------------------- update
    def _accumulate(self, attn_weights: torch.Tensor, num: int) -> None:
        """Fold the new weights ``(B, G, current_length)`` into the score buffers."""
        raise NotImplementedError

    def _compute_scores(self) -> Tuple[torch.Tensor, Dict]:
        """Returns the score tensor ``(B, G, C)`` used for selection and keyword
        arguments for :func:`ops.h2o_update` (normalisation)."""
        raise NotImplementedError

    def _update(self, attn_weights: torch.Tensor, num: int) -> None:
        B = self.batch_size
        L, C = self.current_length, self.cache_length
        if attn_weights.shape != (B, self.n_query_groups, L):
            raise ValueError(f"attn_weights.shape = {tuple(attn_weights.shape)}, must be {(B, self.n_query_groups, L)}")
        self._select_after_accumulate(attn_weights.detach(), num)

    def _select_after_accumulate(self, attn_weights: torch.Tensor, num: int) -> None:
        L, C = self.current_length, self.cache_length
        self._accumulate(attn_weights, num)
        if L < C:
            self._next_positions = None  # free slots are used while filling
            return
        k = self.max_chunk_size if self.max_chunk_size is not None else C - self.grace_period
        self._next_positions = self._select(k)

    def _select(self, k: int) -> torch.Tensor:
        raise NotImplementedError

    def size_estimate(self):
        sz, d = super().size_estimate()
        sc = len(self._score_buffer_names()) * self.max_batch_size * self.n_query_groups * self.cache_length * 32
        return sz + sc, dict(d, scores=sc)

    @classmethod
    def size_estimate_apriori(cls, params: KVCacheParams, **kwargs):
        sz, d = super().size_estimate_apriori(params, **kwargs)
        sc = cls._num_score_buffers() * params.max_batch_size * params.n_query_groups * params.cache_length * 32
        return sz + sc, dict(d, scores=sc)

    @classmethod
    def _num_score_buffers(cls) -> int:
        return 0
