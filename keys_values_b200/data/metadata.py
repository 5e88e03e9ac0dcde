"""Token-length metadata shared by the dataset modules: one JSON file per dataset under ``metadata_dir`` whose nested
keys end in the list of prompt lengths (in tokens) of all records, so that a later run with the same dataset and
tokenizer filters by length without tokenizing again (``keys_values/data/module.py:107-283``)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

METADATA_SEQ_LENGTHS_KEY = "seq_lengths"


def get_nested(d: Optional[Dict[str, Any]], keys: Sequence[str]) -> Any:
    for k in keys:
        if not isinstance(d, dict) or k not in d:
            return None
        d = d[k]
    return d


def set_nested(d: Dict[str, Any], keys: Sequence[str], value: Any) -> None:
    for k in keys[:-1]:
        d = d.setdefault(k, {})
    d[keys[-1]] = value


class LengthMetadata:
    def __init__(self, metadata_dir: Optional[str], file_name: str):
        self.path = None if metadata_dir is None else Path(metadata_dir) / file_name
        self._data: Optional[Dict[str, Any]] = None

    def load(self) -> Dict[str, Any]:
        if self._data is None:
            self._data = {}
            if self.path is not None and self.path.is_file():
                self._data = json.loads(self.path.read_text())
        return self._data

    def lengths(self, keys: Sequence[str], expected: Optional[int] = None) -> Optional[List[int]]:
        got = get_nested(self.load(), [METADATA_SEQ_LENGTHS_KEY, *keys])
        if got is None or (expected is not None and len(got) != expected):
            return None
        return [int(x) for x in got]

    def store(self, keys: Sequence[str], lengths: List[int]) -> None:
        set_nested(self.load(), [METADATA_SEQ_LENGTHS_KEY, *keys], [int(x) for x in lengths])
        if self.path is not None:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            self.path.write_text(json.dumps(self._data))
