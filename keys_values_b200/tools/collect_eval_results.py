"""Reduce the per-batch CSV files written by ``eval_long`` / ``eval_long_ext`` into one table
(``keys_values/scripts/collect_eval_results.py``, ``create_result_table.py``).

    python -m keys_values_b200.tools.collect_eval_results OUT_DIR [OUT_DIR ...] [--eval_dir eval] [--out table.csv]
        [--expected_batches N] [--markdown]

One row per (run, task): token-weighted mean loss and perplexity, the mean of every sample metric that the batch
files carry (columns other than the bookkeeping ones), the number of batch files and rows, the evaluation time,
and, with ``--expected_batches``, whether the task is complete; batches that another worker still holds (a lock
file without a result) are counted as pending. Rows are sorted by run, cache setup and checkpoint step.
"""
from __future__ import annotations

import argparse
import csv
import math
import re
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional

BOOKKEEPING = {"task", "batch", "row", "loss", "num_tokens", "time", "idx", "prompt_length"}


def _step_of(checkpoint: str) -> int:
    m = re.search(r"(\d+)", checkpoint)
    return int(m.group(1)) if m else (1 << 60 if checkpoint == "final" else -1)


def collect(out_dir: Path, eval_dir: str = "eval", expected_batches: Optional[int] = None) -> List[Dict]:
    out_dir = Path(out_dir)
    per_task = defaultdict(lambda: dict(loss=0.0, tokens=0.0, rows=0, files=0, time=0.0, metrics=defaultdict(lambda: [0.0, 0]), pending=0))
    for task_dir in sorted(p for p in out_dir.glob(f"*/{eval_dir}") if p.is_dir()):
        key = task_dir.parent.name
        acc = per_task[key]
        done = set()
        for f in task_dir.glob("eval_metrics_*.csv"):
            acc["files"] += 1
            done.add(f.stem.rsplit("_", 1)[-1])
            with open(f) as fp:
                for row in csv.DictReader(fp):
                    n = float(row.get("num_tokens") or 1)
                    if row.get("loss") not in (None, ""):
                        acc["loss"] += float(row["loss"]) * n
                        acc["tokens"] += n
                    acc["rows"] += 1
                    acc["time"] += float(row.get("time") or 0.0)
                    for col, val in row.items():
                        if col not in BOOKKEEPING and val not in (None, ""):
                            try:
                                m = acc["metrics"][col]
                                m[0] += float(val)
                                m[1] += 1
                            except ValueError:
                                pass
        acc["pending"] = sum(1 for l in task_dir.glob("batch_*.lock") if l.stem.rsplit("_", 1)[-1] not in done)
    rows = []
    for key, acc in per_task.items():
        setup, _, checkpoint = key.partition("__")
        mean = acc["loss"] / acc["tokens"] if acc["tokens"] else float("nan")
        row = {"run": out_dir.name, "setup": setup, "checkpoint": checkpoint, "task": key, "mean_loss": mean,
               "perplexity": math.exp(mean) if mean == mean and mean < 50 else float("nan"), "rows": acc["rows"], "batches": acc["files"],
               "pending_batches": acc["pending"], "eval_time_s": acc["time"]}
        if expected_batches is not None:
            row["complete"] = acc["files"] >= expected_batches
        for col, (total, n) in sorted(acc["metrics"].items()):
            row[col] = total / max(n, 1)
        rows.append(row)
    rows.sort(key=lambda r: (r["run"], r["setup"], _step_of(r["checkpoint"])))
    return rows


def best_checkpoint(rows: List[Dict], by: str = "mean_loss", lower_is_better: bool = True) -> Dict[str, Dict]:
    """Per (run, setup) the row of the best checkpoint."""
    best: Dict[str, Dict] = {}
    for r in rows:
        v = r.get(by)
        if v is None or v != v:
            continue
        k = f"{r['run']}/{r['setup']}"
        if k not in best or (v < best[k][by]) == lower_is_better:
            best[k] = r
    return best


def to_markdown(rows: List[Dict]) -> str:
    if not rows:
        return "(no results)"
    cols = list(dict.fromkeys(c for r in rows for c in r if c != "task"))
    fmt = lambda v: f"{v:.4f}" if isinstance(v, float) else str(v)  # noqa: E731
    lines = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    lines += ["| " + " | ".join(fmt(r.get(c, "")) for c in cols) + " |" for r in rows]
    return "\n".join(lines)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("out_dirs", nargs="+")
    ap.add_argument("--eval_dir", default="eval")
    ap.add_argument("--out", default=None, help="write the table as CSV")
    ap.add_argument("--expected_batches", type=int, default=None)
    ap.add_argument("--markdown", action="store_true")
    args = ap.parse_args(argv)
    rows = [r for d in args.out_dirs for r in collect(Path(d), args.eval_dir, args.expected_batches)]
    if args.out:
        cols = list(dict.fromkeys(c for r in rows for c in r))
        with open(args.out, "w", newline="") as fp:
            w = csv.DictWriter(fp, fieldnames=cols)
            w.writeheader()
            w.writerows(rows)
    print(to_markdown(rows) if args.markdown else "\n".join(str(r) for r in rows))
    for k, r in best_checkpoint(rows).items():
        print(f"best of {k}: {r['checkpoint']} (mean loss {r['mean_loss']:.4f})")


if __name__ == "__main__":
    main(sys.argv[1:])
