"""Reduce the per-batch CSV files written by ``eval_long[_ext]`` into one table
(``keys_values/scripts/collect_eval_results.py``): mean loss (token weighted) per task."""
from __future__ import annotations

import csv
import sys
from collections import defaultdict
from pathlib import Path


def collect(out_dir: Path, eval_dir: str = "eval"):
    acc = defaultdict(lambda: [0.0, 0.0, 0])
    for f in Path(out_dir).glob(f"*/{eval_dir}/eval_metrics_*.csv"):
        with open(f) as fp:
            for row in csv.DictReader(fp):
                a = acc[row["task"]]
                n = float(row.get("num_tokens", 1))
                a[0] += float(row["loss"]) * n
                a[1] += n
                a[2] += 1
    return [{"task": k, "mean_loss": v[0] / max(v[1], 1), "rows": v[2]} for k, v in sorted(acc.items())]


if __name__ == "__main__":
    for r in collect(Path(sys.argv[1]), *(sys.argv[2:3])):
        print(r)
