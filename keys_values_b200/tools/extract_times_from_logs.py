"""Scrape step times, throughput, validation losses and evaluation times from the logs of the commands
(``keys_values/scripts/extract_train_times_from_logs.py``, ``extract_eval_times_from_logs.py``,
``extract_valid_loss_from_logs.py``).

    python -m keys_values_b200.tools.extract_times_from_logs LOG_OR_DIR [...] [--out_prefix times] [--skip 1]

A directory stands for the per-rank logs in it (``gpu0.log``, ``gpu1.log``, … as written with ``KEYSVALS_LOG_DIR``):
the time of a step is the maximum over the ranks that logged it (the ranks wait for each other in the gradient
all-reduce), its throughput the sum. Prints mean / median / 90th percentile of the step time (after ``--skip``
warm-up steps) and writes ``<out_prefix>_train.csv`` / ``_val.csv`` when asked.
"""
from __future__ import annotations

import argparse
import csv
import re
import statistics
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, List

STEP_RE = re.compile(r"step (\d+)/(\d+) \| loss ([\d.eE+-]+|nan|inf) \| ([\d.]+) s \| ([\d.]+) tok/s")
VAL_RE = re.compile(r"validation: \{.*'val_loss': ([\d.eE+-]+|nan|inf).*'val_time': ([\d.]+)")
EVAL_RE = re.compile(r"task ([\w.\-]+__[\w.\-]+) batch (\d+).*?([\d.]+) s")
MEM_RE = re.compile(r"peak memory[^\d]*([\d.]+) ?GB", re.IGNORECASE)


def extract(path: Path) -> Dict[str, List[dict]]:
    """Records of one log file."""
    steps, vals, evals, mem = [], [], [], []
    last_step = 0
    for line in Path(path).read_text(errors="replace").splitlines():
        if (m := STEP_RE.search(line)):
            last_step = int(m.group(1))
            steps.append({"step": last_step, "of": int(m.group(2)), "loss": float(m.group(3)), "iter_time": float(m.group(4)),
                          "tokens_per_sec": float(m.group(5))})
        elif (m := VAL_RE.search(line)):
            vals.append({"after_step": last_step, "val_loss": float(m.group(1)), "val_time": float(m.group(2))})
        elif (m := EVAL_RE.search(line)):
            evals.append({"task": m.group(1), "batch": int(m.group(2)), "time": float(m.group(3))})
        if (m := MEM_RE.search(line)):
            mem.append(float(m.group(1)))
    return {"train": steps, "val": vals, "eval": evals, "peak_memory_gb": mem}


def merge_ranks(per_rank: List[Dict[str, List[dict]]]) -> Dict[str, List[dict]]:
    """Step time = maximum over ranks, throughput = sum, loss = mean; validation records of the first rank that has any."""
    by_step = defaultdict(list)
    for rec in per_rank:
        for s in rec["train"]:
            by_step[s["step"]].append(s)
    train = []
    for step in sorted(by_step):
        group = by_step[step]
        train.append({"step": step, "of": group[0]["of"], "ranks": len(group), "loss": sum(g["loss"] for g in group) / len(group),
                      "iter_time": max(g["iter_time"] for g in group), "tokens_per_sec": sum(g["tokens_per_sec"] for g in group)})
    val = next((r["val"] for r in per_rank if r["val"]), [])
    evals = [e for r in per_rank for e in r["eval"]]
    mem = [m for r in per_rank for m in r["peak_memory_gb"]]
    return {"train": train, "val": val, "eval": evals, "peak_memory_gb": mem}


def summarize(train: List[dict], skip: int = 1) -> Dict[str, float]:
    times = [s["iter_time"] for s in train[skip:]] or [s["iter_time"] for s in train]
    if not times:
        return {}
    times_sorted = sorted(times)
    return {"steps": len(times), "mean_s": statistics.fmean(times), "median_s": statistics.median(times),
            "p90_s": times_sorted[min(len(times) - 1, int(0.9 * len(times)))], "min_s": times_sorted[0], "max_s": times_sorted[-1],
            "mean_tokens_per_sec": statistics.fmean(s["tokens_per_sec"] for s in (train[skip:] or train))}


def load(path: Path) -> Dict[str, List[dict]]:
    path = Path(path)
    if path.is_dir():
        files = sorted(path.glob("gpu*.log")) or sorted(path.glob("*.log"))
        return merge_ranks([extract(f) for f in files])
    return merge_ranks([extract(path)])


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--out_prefix", default=None)
    ap.add_argument("--skip", type=int, default=1, help="warm-up steps left out of the statistics")
    args = ap.parse_args(argv)
    for p in args.paths:
        rec = load(Path(p))
        print(f"{p}: {summarize(rec['train'], args.skip)}")
        for v in rec["val"]:
            print(f"  validation after step {v['after_step']}: loss {v['val_loss']:.4f} in {v['val_time']:.1f} s")
        if rec["eval"]:
            per_task = defaultdict(float)
            for e in rec["eval"]:
                per_task[e["task"]] += e["time"]
            for t, s in sorted(per_task.items()):
                print(f"  evaluation of {t}: {s:.1f} s")
        if rec["peak_memory_gb"]:
            print(f"  peak memory: {max(rec['peak_memory_gb']):.1f} GB")
        if args.out_prefix:
            for kind in ("train", "val"):
                if rec[kind]:
                    with open(f"{args.out_prefix}_{Path(p).stem}_{kind}.csv", "w", newline="") as fp:
                        w = csv.DictWriter(fp, fieldnames=list(rec[kind][0]))
                        w.writeheader()
                        w.writerows(rec[kind])


if __name__ == "__main__":
    main(sys.argv[1:])
