"""Host-side profiling switches of the training step.

* :class:`PartProfiler`: ``cProfile`` around the forward or the backward part of a long-context step, statistics
  sorted by cumulative time (role of ``_debug_profile_forward`` / ``_debug_profile_backward`` in
  ``keys_values/kvcache/gradient/main.py:845-907`` and ``:1080-1322``; there the process exits after the first
  report, here that is the option ``exit_after``).
* :func:`nvtx_range`: named ranges on the CUDA timeline (cells, rows of layers, forward, backward), recorded when
  ``KVB200_NVTX=1`` so that a timeline tool shows which kernels belong to which part of the step.
"""
from __future__ import annotations

import contextlib
import cProfile
import io
import os
import pstats
from typing import Dict, Optional

import torch

PARTS = ("forward", "backward", "both")


class PartProfiler:
    def __init__(self, parts: Optional[str], top: int = 40, exit_after: bool = False, stream=None):
        if parts is not None and parts not in PARTS:
            raise ValueError(f"profile_parts = {parts} not supported; must be in {PARTS}")
        self.parts, self.top, self.exit_after, self.stream = parts, top, exit_after, stream
        self.reports: Dict[str, str] = {}
        self._active: Optional[cProfile.Profile] = None

    def wants(self, part: str) -> bool:
        return self.parts is not None and (self.parts == part or self.parts == "both")

    def start(self, part: str) -> None:
        if self.wants(part) and self._active is None:
            self._active = cProfile.Profile()
            self._active.enable()

    def stop(self, part: str, device=None) -> None:
        if not self.wants(part) or self._active is None:
            return
        if device is not None and torch.device(device).type == "cuda":
            torch.cuda.synchronize(device)  # the last launches belong to this part
        self._active.disable()
        buf = io.StringIO()
        pstats.Stats(self._active, stream=buf).sort_stats(pstats.SortKey.CUMULATIVE).print_stats(self.top)
        self._active = None
        text = f"==== cProfile of the {part} part (cumulative time, top {self.top}) ====\n{buf.getvalue()}"
        self.reports[part] = text
        print(text, file=self.stream, flush=True)
        if self.exit_after and (self.parts != "both" or part == "backward"):
            raise SystemExit(0)


def nvtx_enabled() -> bool:
    return os.environ.get("KVB200_NVTX", "0") == "1" and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if nvtx_enabled():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def nvtx_mark(name: str) -> None:
    """Instantaneous marker on the CUDA timeline (start of a cell of the forward pass, of a row of the backward pass)."""
    if nvtx_enabled():
        torch.cuda.nvtx.mark(name)
