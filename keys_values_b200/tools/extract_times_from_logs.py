"""Scrape per-step times and validation losses from the per-rank logs written by the CLI
(``keys_values/scripts/extract_*_from_logs.py``) into CSV rows."""
from __future__ import annotations

import re
import sys
from pathlib import Path
from typing import Dict, List

STEP_RE = re.compile(r"step (\d+)/(\d+) \| loss ([\d.eE+-]+) \| ([\d.]+) s \| ([\d.]+) tok/s")
VAL_RE = re.compile(r"validation: \{.*'val_loss': ([\d.eE+-]+).*'val_time': ([\d.]+)")


def extract(path: Path) -> Dict[str, List[dict]]:
    steps, vals = [], []
    for line in Path(path).read_text().splitlines():
        if (m := STEP_RE.search(line)):
            steps.append({"step": int(m.group(1)), "loss": float(m.group(3)), "iter_time": float(m.group(4)), "tokens_per_sec": float(m.group(5))})
        elif (m := VAL_RE.search(line)):
            vals.append({"val_loss": float(m.group(1)), "val_time": float(m.group(2))})
    return {"train": steps, "val": vals}


if __name__ == "__main__":
    print(extract(Path(sys.argv[1])))
