"""KV-cache base classes.

A cache owns the position counter: callers never pass positions. One call of
:meth:`KVCache.forward` (1) writes the new keys/values into slots chosen by the
policy, (2) runs SDPA of the new queries against the *updated* cache, masked by
token position, and (3) lets the policy choose the slots for the next call.
Parity: ``keys_values/kvcache/base.py:29-855``.

All policy state (``token_pos``, scores, next slots, replay log) lives in device
tensors and is updated by kernels; nothing in the per-chunk path reads a value
back to the host, so a (layer, chunk) step can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from keys_values_b200.attention.base import DefaultKeysAndValues, KeysAndValues, MultiHeadSelfAttention
from keys_values_b200.config import Config


def bitsize_of(t: torch.Tensor) -> int:
    return t.numel() * t.element_size() * 8


def bits_for_torch_dtype(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size() * 8


@dataclass(frozen=True)
class KVCacheParams:
    max_batch_size: int
    n_query_groups: int
    cache_length: int
    head_size: int
    n_head: int
    dtype: Optional[torch.dtype]

    @staticmethod
    def from_config(config: Config, max_batch_size: int, cache_length: int, dtype=None, head_size=None) -> "KVCacheParams":
        return KVCacheParams(
            max_batch_size=max_batch_size,
            n_query_groups=config.n_query_groups,
            cache_length=cache_length,
            head_size=config.head_size if head_size is None else head_size,
            n_head=config.n_head,
            dtype=dtype,
        )


class KVCache(torch.nn.Module):
    """Abstract cache for one layer."""

    def __init__(self, config: Config, max_batch_size: int, cache_length: int, block_idx: int, dtype=None, head_size=None):
        super().__init__()
        if cache_length <= 0:
            raise ValueError("cache_length must be positive")
        self.config = config
        self.max_batch_size = max_batch_size
        self._n_query_groups = config.n_query_groups
        self._cache_length = cache_length
        self.head_size = config.head_size if head_size is None else head_size
        self.n_head = config.n_head
        self._dtype = dtype
        self.block_idx = block_idx
        self._input_pos = 0
        self._batch_size: Optional[int] = None

    # ---- static properties
    @property
    def cache_length(self) -> int:
        return self._cache_length

    @property
    def n_query_groups(self) -> int:
        return self._n_query_groups

    @property
    def dtype(self):
        return self._dtype

    @property
    def device(self):
        raise NotImplementedError

    def get_params(self) -> KVCacheParams:
        return KVCacheParams(self.max_batch_size, self.n_query_groups, self.cache_length, self.head_size, self.n_head, self.dtype)

    # ---- dynamic state
    @property
    def input_pos(self) -> int:
        """Number of tokens processed since the last :meth:`reset`."""
        return self._input_pos

    @property
    def next_token_pos(self) -> int:
        return self._input_pos

    @property
    def batch_size(self) -> Optional[int]:
        return self._batch_size

    @property
    def current_length(self) -> int:
        raise NotImplementedError

    @property
    def max_prefill_length(self) -> Optional[int]:
        raise NotImplementedError

    def max_forward_length(self) -> int:
        raise NotImplementedError

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, token_idx: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def token_positions(self) -> torch.Tensor:
        """``(B, G, current_length)`` int32: token position held by every slot."""
        raise NotImplementedError

    def get_keys_values(self) -> Optional[KeysAndValues]:
        raise NotImplementedError

    def reset(self) -> None:
        self._input_pos = 0
        self._batch_size = None

    def set_seq_length(self, value: int) -> None:
        pass

    def size_estimate(self) -> Tuple[int, Dict[str, int]]:
        raise NotImplementedError

    @classmethod
    def size_estimate_apriori(cls, params: KVCacheParams, **kwargs) -> Tuple[int, Dict[str, int]]:
        raise NotImplementedError

    def clone(self, device=None) -> "KVCache":
        raise NotImplementedError

    def switch_replay_logging(self, status: bool) -> None:
        pass

    def get_replay_log(self) -> Optional["KVCacheReplayLog"]:
        return None


class KVCacheReplayLog:
    """Everything needed to replay the insert decisions of one cache: the chunk
    sizes in order, and for every non-prefill chunk the slots ``(B, G, n)`` int32
    its tokens were written to (kept on the device of the cache)."""

    def __init__(self, cache_length: int, grace_period: int = 0):
        self.cache_length = cache_length
        self.grace_period = grace_period
        self.token_chunks: List[int] = []
        self.slot_positions: List[Optional[torch.Tensor]] = []

    def append(self, num: int, slots: Optional[torch.Tensor]) -> None:
        self.token_chunks.append(num)
        self.slot_positions.append(slots)

    def __len__(self) -> int:
        return sum(self.token_chunks)

    def chunk_starts(self) -> List[int]:
        starts, s = [], 0
        for n in self.token_chunks:
            starts.append(s)
            s += n
        return starts

    def slots_for(self, token_pos: int, num: int) -> Optional[torch.Tensor]:
        """Slots of the chunk that starts at ``token_pos`` with ``num`` tokens."""
        s = 0
        for n, slots in zip(self.token_chunks, self.slot_positions):
            if s == token_pos:
                if n != num:
                    raise IndexError(f"chunk at {token_pos} has {n} tokens, not {num}")
                return slots
            s += n
        raise IndexError(f"No chunk starts at token position {token_pos}")


class DefaultKVCache(KVCache):
    """Cache whose forward is ``write → SDPA → policy update``
    (``keys_values/kvcache/base.py:403-712``)."""

    def __init__(self, config, max_batch_size, cache_length, block_idx, dtype=None, head_size=None, mha: Optional[MultiHeadSelfAttention] = None, **mha_kwargs):
        super().__init__(config, max_batch_size, cache_length, block_idx, dtype, head_size)
        self.mha = mha if mha is not None else MultiHeadSelfAttention(config, **mha_kwargs)
        # ``recorder(block_idx, input_pos, attn_out, lse)``: set by the training forward
        # pass to keep attention outputs and normalisers for the backward pass
        self.attn_recorder = None

    def set_seq_length(self, value: int) -> None:
        self.mha.set_seq_length(value)

    def needs_attn_weights(self) -> bool:
        return False

    # -- to be provided by subclasses
    def _prefill(self, key: torch.Tensor, value: torch.Tensor, token_idx: torch.Tensor) -> None:
        raise NotImplementedError

    def _forward(self, key: torch.Tensor, value: torch.Tensor, token_idx: torch.Tensor) -> KeysAndValues:
        raise NotImplementedError

    def _update(self, *args, **kwargs) -> None:
        pass

    def advance_host_counters(self) -> None:
        """One token has been processed by a captured decode step: move the host counters on."""
        self._input_pos += 1

    def _can_decode_direct(self, query: torch.Tensor) -> bool:
        """True if a single new token can be served by the decode kernel that reads
        the cache storage directly (quantized storage included)."""
        return False

    def _decode_direct(self, query, key, value, token_idx, need_weights: bool):
        raise NotImplementedError

    def _check_args(self, query, key, value, token_idx) -> int:
        if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
            raise ValueError("query, key, value must be 4D")
        B, H, n, D = query.shape
        if key.shape != value.shape or key.shape != (B, self.n_query_groups, n, self.head_size) or H != self.n_head or D != self.head_size:
            raise ValueError(
                f"shapes query {tuple(query.shape)}, key {tuple(key.shape)}, value {tuple(value.shape)} inconsistent with "
                f"n_head={self.n_head}, n_query_groups={self.n_query_groups}, head_size={self.head_size}"
            )
        if token_idx is not None and tuple(token_idx.shape) != (B, n):
            raise ValueError(f"token_idx.shape = {tuple(token_idx.shape)}, must be {(B, n)}")
        if self._input_pos == 0:
            if B > self.max_batch_size:
                raise ValueError(f"batch size {B} > max_batch_size {self.max_batch_size}")
            mpl = self.max_prefill_length
            if mpl is not None and n > mpl:
                raise ValueError(f"prefill length {n} > max_prefill_length {mpl}")
        else:
            if B != self._batch_size:
                raise ValueError(f"batch size {B} differs from the one used in prefill ({self._batch_size})")
            if n > self.max_forward_length():
                raise ValueError(f"query length {n} > max_forward_length {self.max_forward_length()}")
        return n

    def forward(self, query, key, value, token_idx):
        n = self._check_args(query, key, value, token_idx)
        if self._input_pos == 0:
            self._batch_size = query.shape[0]
            self._prefill(key, value, token_idx)
            if self.attn_recorder is not None:
                attn_out, _, lse = self.mha(query, DefaultKeysAndValues(key, value), block_idx=self.block_idx, input_pos=0, return_lse=True)
                self.attn_recorder(self.block_idx, 0, attn_out, lse)
            else:
                attn_out, _ = self.mha(query, DefaultKeysAndValues(key, value), block_idx=self.block_idx, input_pos=0)
            self._input_pos = n
            return attn_out
        input_pos = self._input_pos
        need_w = self.needs_attn_weights()
        if n == 1 and self.attn_recorder is None and self._can_decode_direct(query):
            attn_out, weights = self._decode_direct(query, key, value, token_idx, need_w)
            self._input_pos = input_pos + 1
            if need_w:
                self._update(weights, 1)
            return attn_out
        k_and_v = self._forward(key, value, token_idx)
        if self.attn_recorder is not None:
            attn_out, weights, lse = self.mha(
                query, k_and_v, block_idx=self.block_idx, input_pos=input_pos,
                return_attn_weights=need_w, token_positions=self.token_positions(), return_lse=True,
            )
            self.attn_recorder(self.block_idx, input_pos, attn_out, lse)
        else:
            attn_out, weights = self.mha(
                query, k_and_v, block_idx=self.block_idx, input_pos=input_pos,
                return_attn_weights=need_w, token_positions=self.token_positions(),
            )
        self._input_pos = input_pos + n
        if need_w:
            self._update(weights, n)
        return attn_out
