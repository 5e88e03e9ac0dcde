"""Out-of-memory retry ladder for the long-context forward / backward.

A step is attempted with the largest temporary-array limit and with the attention outputs of the
forward pass kept for the backward pass. On ``torch.OutOfMemoryError`` the caller's ``free_fn``
releases what can be released (autograd arrays, the allocator cache); the next attempt first gives
up the saved attention outputs (they are recomputed in the backward pass instead), then walks down
the ladder of limits. Parity: ``oom_exception_action`` in ``keys_values/long_context.py:333-363``
and the ladder of ``keys_values/array_limit.py:29-64``.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch


class OOMRetry:
    def __init__(self, limits_gb: Sequence[float], free_fn: Optional[Callable[[], None]] = None, verbose: bool = False):
        if not limits_gb:
            raise ValueError("limits_gb must not be empty")
        self.limits_gb = tuple(limits_gb)
        self.free_fn = free_fn if free_fn is not None else self._default_free
        self.verbose = verbose
        self.attempts = 0

    @staticmethod
    def _default_free() -> None:
        import gc

        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def ladder(self):
        """(limit_gb, save_attention_outputs) in the order in which they are tried."""
        yield self.limits_gb[0], True
        for lim in self.limits_gb:
            yield lim, False

    def run(self, step_fn: Callable[[float, bool], object]):
        last = None
        for limit_gb, save_attention in self.ladder():
            self.attempts += 1
            try:
                return step_fn(limit_gb, save_attention)
            except torch.OutOfMemoryError as ex:  # noqa: PERF203
                last = ex
                if self.verbose:
                    print(f"out of memory with limit {limit_gb} GB, save_attention_outputs={save_attention}: retrying")
                self.free_fn()
        raise last
