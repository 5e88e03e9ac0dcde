"""House-keeping for the output directories of fine-tuning and evaluation runs.

    python -m keys_values_b200.tools.experiment_files <command> <dir> [options]

    cleanup-evaluation   remove lock files left by stopped evaluation workers (``--results``: the results too)
    cleanup-gen-samples  remove the per-batch files of generated samples
    collect-gen-samples  join the per-batch sample files of every task into ``generated_samples_all.yaml``
    convert-samples      ``evaluation.jsonl`` (one JSON object per sample) → the YAML sample format
    sample-stats         length and score statistics of generated samples per task (CSV on stdout)
    collect-val-loss     validation losses of a fine-tuning run (``metrics.csv``) → ``val_losses.yaml``
    result-table         all ``eval_metrics_*.csv`` of a run → ``eval_metrics_all.csv`` and a table per task
    strip-checkpoints    delete what intermediate checkpoints do not need to be evaluated (training state,
                         copied tokenizer files), keeping weights and configuration

One tool instead of the reference's collection of scripts with hard-wired experiment paths
(``keys_values/scripts/{cleanup_evaluation, cleanup_gen_samples, collect_gen_samples,
convert_generated_samples, stats_on_generated_samples, collect_val_loss_yaml, create_result_table,
remove_files_from_checkpoints}.py``); file names are those this framework writes.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import sys
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, Iterable, List

import yaml

SAMPLES_GLOB = "generated_samples_[0-9]*.yaml"
SAMPLES_ALL = "generated_samples_all.yaml"
METRICS_ALL = "eval_metrics_all.csv"
REMOVABLE_FROM_CHECKPOINTS = ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "generation_config.json", "training_state.pth",
                              "training_state.pt", "optimizer.pt")


def _task_dirs(out_dir: Path, eval_dir: str) -> List[Path]:
    return sorted(p for p in Path(out_dir).glob(f"*/{eval_dir}") if p.is_dir())


def _read_samples(path: Path) -> List[Dict[str, Any]]:
    return [d for d in yaml.safe_load_all(path.read_text()) if d]


def _write_samples(path: Path, docs: Iterable[Dict[str, Any]]) -> None:
    with open(path, "w") as fp:
        for d in docs:
            fp.write(yaml.safe_dump(d) + "---\n")


def cleanup_evaluation(out_dir: Path, eval_dir: str = "eval", results: bool = False) -> int:
    n = 0
    for d in _task_dirs(out_dir, eval_dir):
        for f in list(d.glob("batch_*.lock")) + (list(d.glob("eval_metrics_*.csv")) if results else []):
            f.unlink()
            n += 1
    return n


def cleanup_gen_samples(out_dir: Path, eval_dir: str = "eval") -> int:
    n = 0
    for d in _task_dirs(out_dir, eval_dir):
        for f in d.glob(SAMPLES_GLOB):
            f.unlink()
            n += 1
    return n


def collect_gen_samples(out_dir: Path, eval_dir: str = "eval") -> Dict[str, int]:
    counts = {}
    for d in _task_dirs(out_dir, eval_dir):
        files = sorted(d.glob(SAMPLES_GLOB), key=lambda f: int(f.stem.rsplit("_", 1)[1]))
        docs = []
        for f in files:
            for i, doc in enumerate(_read_samples(f)):
                docs.append({"batch": int(f.stem.rsplit("_", 1)[1]), "row": i, **doc})
        if docs:
            _write_samples(d / SAMPLES_ALL, docs)
            counts[d.parent.name] = len(docs)
    return counts


def convert_samples(jsonl: Path, target: Path) -> int:
    docs = []
    for line in jsonl.read_text().splitlines():
        if line.strip():
            rec = json.loads(line)
            docs.append({"reference": rec.get("reference", rec.get("answer", rec.get("output", ""))),
                         "generated": rec.get("generated", rec.get("prediction", rec.get("response", "")))})
    _write_samples(target, docs)
    return len(docs)


def _mean_std(xs: List[float]):
    if not xs:
        return float("nan"), float("nan")
    m = sum(xs) / len(xs)
    return m, math.sqrt(sum((x - m) ** 2 for x in xs) / len(xs))


def sample_stats(out_dir: Path, eval_dir: str = "eval") -> List[Dict[str, Any]]:
    rows = []
    for d in _task_dirs(out_dir, eval_dir):
        docs = _read_samples(d / SAMPLES_ALL) if (d / SAMPLES_ALL).is_file() else [x for f in sorted(d.glob(SAMPLES_GLOB)) for x in _read_samples(f)]
        if not docs:
            continue
        gen = [len(str(x.get("generated", "")).split()) for x in docs]
        ref = [len(str(x.get("reference", "")).split()) for x in docs]
        ratio = [g / max(r, 1) for g, r in zip(gen, ref)]
        scores = [float(x["score"]) for x in docs if "score" in x]
        (gm, gs), (rm, rs), (qm, qs) = _mean_std(gen), _mean_std(ref), _mean_std(ratio)
        rows.append({"task": d.parent.name, "samples": len(docs), "generated_words_mean": gm, "generated_words_std": gs, "reference_words_mean": rm,
                     "reference_words_std": rs, "length_ratio_mean": qm, "length_ratio_std": qs, "empty_generations": sum(g == 0 for g in gen),
                     "score_mean": _mean_std(scores)[0]})
    return rows


def collect_val_loss(out_dir: Path) -> Dict[int, float]:
    losses: Dict[int, float] = {}
    for f in [Path(out_dir) / "metrics.csv"] + sorted(Path(out_dir).glob("logs/**/metrics.csv")):
        if not f.is_file():
            continue
        with open(f) as fp:
            for row in csv.DictReader(fp):
                if row.get("val_loss") not in (None, ""):
                    losses[int(float(row.get("step", 0)))] = float(row["val_loss"])
    if losses:
        (Path(out_dir) / "val_losses.yaml").write_text(yaml.safe_dump({"val_loss": {int(k): float(v) for k, v in sorted(losses.items())}}))
    return losses


def result_table(out_dir: Path, eval_dir: str = "eval") -> List[Dict[str, Any]]:
    all_rows: List[Dict[str, Any]] = []
    for d in _task_dirs(out_dir, eval_dir):
        for f in sorted(d.glob("eval_metrics_[0-9]*.csv")):
            with open(f) as fp:
                all_rows.extend(csv.DictReader(fp))
    if not all_rows:
        return []
    fields = sorted({k for r in all_rows for k in r})
    with open(Path(out_dir) / METRICS_ALL, "w", newline="") as fp:
        w = csv.DictWriter(fp, fieldnames=fields)
        w.writeheader()
        w.writerows(all_rows)
    acc: Dict[str, Dict[str, List[float]]] = defaultdict(lambda: defaultdict(list))
    weights: Dict[str, List[float]] = defaultdict(list)
    for r in all_rows:
        weights[r["task"]].append(float(r.get("num_tokens") or 1))
        for k, v in r.items():
            if k in ("task", "batch", "row", "num_tokens") or v in (None, ""):
                continue
            acc[r["task"]][k].append(float(v))
    table = []
    for task in sorted(acc):
        row: Dict[str, Any] = {"task": task, "rows": len(weights[task])}
        for k, vals in sorted(acc[task].items()):
            if k == "loss" and len(vals) == len(weights[task]):  # token-weighted
                row[k] = sum(v * w for v, w in zip(vals, weights[task])) / sum(weights[task])
            elif k == "time":
                row[k] = sum(vals)
            else:
                row[k] = sum(vals) / len(vals)
        table.append(row)
    return table


def strip_checkpoints(base: Path, keep: Iterable[str] = ("final",)) -> int:
    n = 0
    for step_dir in sorted(Path(base).glob("**/step-*")):
        if not step_dir.is_dir() or step_dir.name in keep:
            continue
        for name in REMOVABLE_FROM_CHECKPOINTS:
            f = step_dir / name
            if f.is_file():
                f.unlink()
                n += 1
    return n


def _print_table(rows: List[Dict[str, Any]]) -> None:
    if not rows:
        print("nothing found")
        return
    fields = list(dict.fromkeys(k for r in rows for k in r))
    w = csv.DictWriter(sys.stdout, fieldnames=fields)
    w.writeheader()
    for r in rows:
        w.writerow({k: (f"{v:.4g}" if isinstance(v, float) else v) for k, v in r.items()})


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("command", choices=["cleanup-evaluation", "cleanup-gen-samples", "collect-gen-samples", "convert-samples", "sample-stats",
                                        "collect-val-loss", "result-table", "strip-checkpoints"])
    ap.add_argument("path", type=Path)
    ap.add_argument("--eval-dir", default="eval")
    ap.add_argument("--results", action="store_true", help="cleanup-evaluation: remove the result files too")
    ap.add_argument("--target", type=Path, default=None, help="convert-samples: output file")
    a = ap.parse_args(argv)
    if a.command == "cleanup-evaluation":
        print(f"removed {cleanup_evaluation(a.path, a.eval_dir, a.results)} files")
    elif a.command == "cleanup-gen-samples":
        print(f"removed {cleanup_gen_samples(a.path, a.eval_dir)} files")
    elif a.command == "collect-gen-samples":
        print(collect_gen_samples(a.path, a.eval_dir))
    elif a.command == "convert-samples":
        print(f"converted {convert_samples(a.path, a.target or a.path.with_name('generated_samples_0.yaml'))} samples")
    elif a.command == "sample-stats":
        _print_table(sample_stats(a.path, a.eval_dir))
    elif a.command == "collect-val-loss":
        print(collect_val_loss(a.path))
    elif a.command == "result-table":
        _print_table(result_table(a.path, a.eval_dir))
    else:
        print(f"removed {strip_checkpoints(a.path)} files")


if __name__ == "__main__":
    main()
