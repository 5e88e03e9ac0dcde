"""GPU memory snapshots around training phases (``keys_values/gpu_memory.py:24-79``): wraps
``torch.cuda.memory._record_memory_history`` / ``_dump_snapshot``; each ``start(name)`` …
``stop()`` pair writes ``<dir>/<name>.pickle`` that https://pytorch.org/memory_viz can open."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch


class RecordGPUMemory:
    def __init__(self, path: Path, max_entries: int = 100000, verbose: bool = False):
        self.path, self.max_entries, self.verbose = Path(path), max_entries, verbose
        self._name: Optional[str] = None

    @property
    def is_recording(self) -> bool:
        return self._name is not None

    def start(self, name: str) -> None:
        if not torch.cuda.is_available():
            return
        self.path.mkdir(parents=True, exist_ok=True)
        torch.cuda.memory._record_memory_history(max_entries=self.max_entries)
        self._name = name

    def stop(self) -> None:
        if self._name is None:
            return
        try:
            torch.cuda.memory._dump_snapshot(str(self.path / f"{self._name}.pickle"))
        finally:
            torch.cuda.memory._record_memory_history(enabled=None)
            self._name = None
