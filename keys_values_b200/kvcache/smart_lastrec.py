"""Last-recently-inserted cache with a per-row protected initial part.

For each batch row the end of the "initial part" (typically the system prompt)
is located by a regular expression on the decoded prompt; the slots that hold it
are never overwritten, the remaining slots form a ring. Parity:
``keys_values/kvcache/smart_lastrec.py:41-771``.

The ring order of every row is computed once at prefill on the host (it depends
on decoded text); afterwards the slots of each forward call are produced by a
gather on the device, so the per-chunk path stays free of host synchronisation.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple, Union

import torch

from keys_values_b200.attention.base import KeysAndValues
from keys_values_b200.kvcache.basics import KVCacheWithBuffers


@dataclass(frozen=True)
class SmartInitialInformation:
    end_initial_regex: Union[str, re.Pattern]
    max_initial_fraction: float
    include_end_string: bool = True

    def __post_init__(self):
        if self.max_initial_fraction == 0:
            raise ValueError("Use LastRecentlyInsertedKVCache for cache without initial parts")
        if not (0 < self.max_initial_fraction < 1):
            raise ValueError(f"max_initial_fraction = {self.max_initial_fraction}, must be in (0, 1)")


def end_initial_regex_from_string(s: str, tokenizer, do_escape: bool = True) -> str:
    """Round-trip ``s`` through the tokenizer so that it matches decoded text."""
    ids = tokenizer.encode(s)
    ids = ids.tolist() if hasattr(ids, "tolist") else list(getattr(ids, "ids", ids))
    result = tokenizer.decode(ids)
    return re.escape(result) if do_escape else result


def find_initial_part(
    token_ids: List[int], tokenizer, regex: Union[str, re.Pattern], include_end_string: bool = True, pad_id: Optional[int] = None
) -> Optional[Tuple[int, int]]:
    """Token range ``[start, end)`` of the initial part of one prompt, or ``None`` if
    the regex does not match. Leading ``pad_id`` tokens are skipped."""
    start = 0
    if pad_id is not None:
        while start < len(token_ids) and token_ids[start] == pad_id:
            start += 1
    ids = token_ids[start:]
    text = tokenizer.decode(ids)
    m = re.search(regex, text)
    if m is None:
        return None
    char_end = m.end() if include_end_string else m.start()
    if char_end <= 0:
        return None
    # smallest number of tokens whose decoding covers char_end characters
    lo, hi = 1, len(ids)
    while lo < hi:
        mid = (lo + hi) // 2
        if len(tokenizer.decode(ids[:mid])) >= char_end:
            hi = mid
        else:
            lo = mid + 1
    return start, start + lo


class SmartInitialLastRecentlyInsertedKVCache(KVCacheWithBuffers):
    def __init__(
        self,
        config,
        buffers,
        block_idx: int,
        tokenizer: Any = None,
        end_initial_regex: Union[str, re.Pattern, None] = None,
        max_initial_fraction: float = 0.25,
        include_end_string: bool = True,
        pad_id: Optional[int] = None,
        **base_kwargs,
    ):
        super().__init__(config, buffers, block_idx, **base_kwargs)
        self.tokenizer = tokenizer
        self.info = None if end_initial_regex is None else SmartInitialInformation(end_initial_regex, max_initial_fraction, include_end_string)
        self.pad_id = pad_id
        self.protected: List[Optional[Tuple[int, int]]] = []
        self._ring: Optional[torch.Tensor] = None  # (B, C) int32 ring order, padded
        self._ring_len: Optional[torch.Tensor] = None  # (B,) int64
        self._ptr: Optional[torch.Tensor] = None  # (B,) int64 position in the ring
        self._min_ring = buffers.cache_length

    def max_forward_length(self) -> int:
        diff = self.cache_length - self.current_length
        return diff if diff > 0 else self._min_ring

    def _protected_ranges(self, token_idx: torch.Tensor) -> List[Optional[Tuple[int, int]]]:
        B, n = token_idx.shape
        if self.info is None or self.tokenizer is None:
            return [None] * B
        cap = int(self.info.max_initial_fraction * self.cache_length)
        rows = token_idx.tolist()
        out = []
        for ids in rows:
            r = find_initial_part(ids, self.tokenizer, self.info.end_initial_regex, self.info.include_end_string, self.pad_id)
            if r is not None:
                s, e = r
                e = min(e, s + cap, n)
                r = (s, e) if e > s else None
            out.append(r)
        return out

    def _prefill(self, key, value, token_idx) -> None:
        super()._prefill(key, value, token_idx)
        B, C, n = key.shape[0], self.cache_length, key.shape[2]
        self.protected = self._protected_ranges(token_idx)
        ring = torch.zeros((B, C), dtype=torch.int32)
        lens, ptrs = [], []
        for b, r in enumerate(self.protected):
            order = [s for s in range(C) if r is None or not (r[0] <= s < r[1])]
            ring[b, : len(order)] = torch.tensor(order, dtype=torch.int32)
            lens.append(len(order))
            # next write goes to slot n (if free) else to the oldest unprotected slot
            ptrs.append(order.index(n) if n < C else 0)
        self._ring = ring.to(key.device)
        self._ring_len = torch.tensor(lens, dtype=torch.int64, device=key.device)
        self._ptr = torch.tensor(ptrs, dtype=torch.int64, device=key.device)
        self._min_ring = min(lens)

    def _forward(self, key, value, token_idx) -> KeysAndValues:
        B, _, n, _ = key.shape
        C = self.cache_length
        L = self.current_length
        if L < C and n > C - L:
            raise ValueError(f"key.shape[2] = {n}, must be <= {C - L} as long as the cache is not full")
        off = (self._ptr.unsqueeze(1) + torch.arange(n, device=key.device)) % self._ring_len.unsqueeze(1)
        slots = self._ring.gather(1, off).unsqueeze(1).expand(B, self.n_query_groups, n).contiguous()
        self.kv_buffers.write(slots, key, value, self.token_pos, self.input_pos)
        self._ptr = (self._ptr + n) % self._ring_len
        if L < C:
            self.kv_buffers.grow(L + n)
        self._log(n, slots)
        return self.kv_buffers.get_keys_values()

    def reset(self) -> None:
        super().reset()
        self.protected = []
        self._ring = self._ring_len = self._ptr = None
        self._min_ring = self.cache_length
