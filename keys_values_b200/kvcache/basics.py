"""Caches that need no attention weights: dense and last-recently-inserted.

Parity: ``keys_values/kvcache/basics.py:39-721``.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from keys_values_b200 import ops
from keys_values_b200.attention.base import KeysAndValues
from keys_values_b200.config import Config
from keys_values_b200.kvcache.base import DefaultKVCache, KVCacheParams, KVCacheReplayLog
from keys_values_b200.kvcache.buffers import DefaultKVCacheBuffers, KVCacheBuffers, KVCacheBuffersParams


class KVCacheWithBuffers(DefaultKVCache):
    """Cache = policy + :class:`KVCacheBuffers` + ``token_pos (B,G,C)`` int32."""

    def __init__(self, config: Config, buffers: KVCacheBuffers, block_idx: int, **base_kwargs):
        super().__init__(
            config, buffers.max_batch_size, buffers.cache_length, block_idx,
            dtype=buffers.dtype, head_size=buffers.head_size, **base_kwargs,
        )
        self.kv_buffers = buffers
        self.token_pos: Optional[torch.Tensor] = None
        self._replay_log: Optional[KVCacheReplayLog] = None
        self._do_replay_log = False

    @classmethod
    def from_config(cls, config: Config, max_batch_size: int, cache_length: int, block_idx: int, device=None, dtype=None, head_size=None, **kwargs):
        params = KVCacheBuffersParams(
            max_batch_size, config.n_query_groups, config.head_size if head_size is None else head_size, dtype, device
        )
        return cls(config, DefaultKVCacheBuffers(params, cache_length), block_idx, **kwargs)

    @property
    def device(self):
        return self.kv_buffers.device

    @property
    def dtype(self):
        return self.kv_buffers.dtype

    @property
    def current_length(self) -> int:
        return self.kv_buffers.current_length

    @property
    def max_prefill_length(self) -> Optional[int]:
        return self.cache_length

    def _alloc_token_pos(self, device) -> None:
        if self.token_pos is None or self.token_pos.device != torch.device(device):
            with torch.inference_mode(False):
                self.token_pos = torch.zeros((self.max_batch_size, self.n_query_groups, self.cache_length), dtype=torch.int32, device=device)

    def token_positions(self) -> torch.Tensor:
        return self.token_pos[: self.batch_size, :, : self.current_length]

    def get_keys_values(self) -> Optional[KeysAndValues]:
        return self.kv_buffers.get_keys_values() if self.current_length > 0 else None

    def reset(self) -> None:
        super().reset()
        self.kv_buffers.reset()
        self._replay_log = None

    # -- single-token decode straight from the storage
    def _can_decode_direct(self, query: torch.Tensor) -> bool:
        if not query.is_cuda or (torch.is_grad_enabled() and query.requires_grad):
            return False
        from keys_values_b200.ops import cuda as _cu

        return _cu.decode_supported(query, self.n_query_groups) and self.kv_buffers.supports_direct_decode()

    def _decode_direct(self, query, key, value, token_idx, need_weights: bool):
        self.kv_buffers.decode_mode = True
        try:
            self._forward(key, value, token_idx)
        finally:
            self.kv_buffers.decode_mode = False
        # a layer with a sliding window hides the slots whose token has left it; capped scores go through tanh in the kernel
        window = self.mha.sliding_window(self.block_idx)
        variant = dict(softcap=self.config.attention_logit_softcapping)
        if window is not None:
            variant.update(sliding_window=window, token_pos=self.token_pos, query_pos=self.input_pos)
        return self.kv_buffers.decode_attention(query, self.mha.pos_encoding.sdpa_scale_factor(), need_weights, **variant)

    def deallocate_buffers(self) -> None:
        self.kv_buffers.deallocate()

    # -- replay logging
    def switch_replay_logging(self, status: bool) -> None:
        self._do_replay_log = status
        if not status:
            self._replay_log = None

    def get_replay_log(self) -> Optional[KVCacheReplayLog]:
        return self._replay_log

    def _log(self, num: int, slots: Optional[torch.Tensor]) -> None:
        if self._do_replay_log:
            if self._replay_log is None:
                self._replay_log = KVCacheReplayLog(self.cache_length, getattr(self, "grace_period", 0))
            self._replay_log.append(num, None if slots is None else slots.clone())

    # -- common prefill
    def _prefill(self, key, value, token_idx) -> None:
        n = key.shape[2]
        B = key.shape[0]
        self._alloc_token_pos(key.device)
        self.kv_buffers.prefill(key, value)
        self.token_pos[:B, :, :n] = torch.arange(n, dtype=torch.int32, device=key.device)
        self._log(n, None)

    def kv_snapshot(self) -> Dict[str, Any]:
        """State needed to restart a replay at this point: keys/values of the
        occupied slots (quantized storage if the buffers are quantized), the token
        positions, and the counters."""
        snap: Dict[str, Any] = dict(
            input_pos=self.input_pos, current_length=self.current_length, batch_size=self.batch_size,
            token_pos=self.token_positions().clone(),
        )
        if getattr(self, "next_grace_pos", None) is not None:
            snap["next_grace_pos"] = int(self.next_grace_pos)  # oldest entry of the grace ring
        if hasattr(self.kv_buffers, "snapshot"):
            snap["quantized"] = self.kv_buffers.snapshot()
            snap["num_bits"] = self.kv_buffers.num_bits
            snap["blocks_over_heads"] = self.kv_buffers.quantizer_k.blocks_over_heads
        else:
            k, v = self.kv_buffers.get_keys_values().both()
            snap["k"], snap["v"] = k.clone(), v.clone()
        return snap

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        sz, d = self.kv_buffers.size_estimate()
        tp = self.max_batch_size * self.n_query_groups * self.cache_length * 32
        d = dict(d, token_pos=tp)
        return sz + tp, d

    @classmethod
    def size_estimate_apriori(cls, params: KVCacheParams, **kwargs):
        sz, d = DefaultKVCacheBuffers.size_estimate_apriori(params, **kwargs)
        tp = params.max_batch_size * params.n_query_groups * params.cache_length * 32
        return sz + tp, dict(d, token_pos=tp)

    def clone(self, device=None):
        import copy

        mha = self.mha
        self.mha = None
        try:
            other = copy.deepcopy(self)
        finally:
            self.mha = mha
        other.mha = mha
        if device is not None:
            other = other.to(device)
        return other


class DenseKVCache(KVCacheWithBuffers):
    """Append-only cache; an error is raised when it is full
    (``keys_values/kvcache/basics.py:294-435``)."""

    def max_forward_length(self) -> int:
        return self.cache_length - self.current_length

    def _forward(self, key, value, token_idx) -> KeysAndValues:
        n = key.shape[2]
        L = self.current_length
        if L + n > self.cache_length:
            raise IndexError(f"Dense cache is full: {L} + {n} > cache_length {self.cache_length}")
        B = key.shape[0]
        slots = torch.arange(L, L + n, dtype=torch.int32, device=key.device).view(1, 1, n).expand(B, self.n_query_groups, n)
        self.kv_buffers.write(slots, key, value, self.token_pos, self.input_pos)
        self.kv_buffers.grow(L + n)
        self._log(n, slots)
        return self.kv_buffers.get_keys_values()


class LastRecentlyInsertedKVCacheReplayLog(KVCacheReplayLog):
    pass


def default_init_grace_tokens(cache_length: int) -> int:
    return min(16, max(cache_length // 8, 1))


class LastRecentlyInsertedKVCache(KVCacheWithBuffers):
    """Keeps the first ``init_grace_tokens`` tokens (attention sinks) and the most
    recent ones: a ring buffer over slots ``[init_grace_tokens, C)``
    (``keys_values/kvcache/basics.py:498-721``)."""

    def __init__(self, config, buffers, block_idx, init_grace_tokens: Optional[int] = None, **base_kwargs):
        super().__init__(config, buffers, block_idx, **base_kwargs)
        if init_grace_tokens is None:
            init_grace_tokens = default_init_grace_tokens(buffers.cache_length)
        if not (0 <= init_grace_tokens < buffers.cache_length):
            raise ValueError(f"init_grace_tokens = {init_grace_tokens} must be in [0, {buffers.cache_length})")
        self.init_grace_tokens = init_grace_tokens
        self.next_position = 0

    def max_forward_length(self) -> int:
        return self.cache_length - self.init_grace_tokens

    def _ring_start(self, batch_idx=None) -> int:
        return self.init_grace_tokens

    def _prefill(self, key, value, token_idx) -> None:
        super()._prefill(key, value, token_idx)
        n = key.shape[2]
        self.next_position = n if n < self.cache_length else self._ring_start()

    def advance_host_counters(self) -> None:
        """One token has been processed by a captured decode step: move the host counters on."""
        C, s = self.cache_length, self._ring_start()
        self._input_pos += 1
        nxt = self.next_position + 1
        self.next_position = nxt if nxt < C else (nxt - C) % (C - s) + s

    def _next_slots(self, n: int, B: int, device) -> torch.Tensor:
        L, C, s = self.current_length, self.cache_length, self._ring_start()
        ctx = ops.position_context() if n == 1 else None
        if ctx is not None:
            # captured decode step of a full cache: the slot follows from the device-resident position
            pos = ctx.word.to(torch.int64)
            slot = (pos - C) % (C - s) + s
            return slot.to(torch.int32).view(1, 1, 1).expand(B, self.n_query_groups, 1)
        pos = torch.arange(n, dtype=torch.int64, device=device) + self.next_position
        # positions past the end wrap into the ring [s, C)
        pos = torch.where(pos < C, pos, (pos - C) % (C - s) + s)
        return pos.to(torch.int32).view(1, 1, n).expand(B, self.n_query_groups, n)

    def _forward(self, key, value, token_idx) -> KeysAndValues:
        n, B = key.shape[2], key.shape[0]
        C, s = self.cache_length, self._ring_start()
        slots = self._next_slots(n, B, key.device)
        self.kv_buffers.write(slots, key, value, self.token_pos, self.input_pos)
        nxt = self.next_position + n
        self.kv_buffers.grow(min(C, max(self.current_length, nxt)))
        self.next_position = nxt if nxt < C else (nxt - C) % (C - s) + s
        self._log(n, slots)
        return self.kv_buffers.get_keys_values()

    def reset(self) -> None:
        super().reset()
        self.next_position = 0
