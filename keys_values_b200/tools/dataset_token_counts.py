"""Token-count statistics of an instruction dataset (``keys_values/scripts/dataset_token_counts.py``).

    python -m keys_values_b200.tools.dataset_token_counts <data.json|jsonl> <checkpoint_dir> [--field instruction --field output]

Prints count, mean and quantiles of the number of tokens per record (the named fields joined by a
newline), so that ``--train.max_seq_length`` and the cache length can be chosen.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Callable, Dict, List, Sequence


def load_records(path: Path) -> List[Dict[str, str]]:
    text = Path(path).read_text()
    if str(path).endswith(".jsonl"):
        return [json.loads(line) for line in text.splitlines() if line.strip()]
    data = json.loads(text)
    return data if isinstance(data, list) else data.get("data", [])


def token_counts(records: Sequence[Dict[str, str]], encode: Callable[[str], Sequence[int]], fields: Sequence[str]) -> List[int]:
    return [len(encode("\n".join(str(r.get(f, "")) for f in fields if r.get(f)))) for r in records]


def summarize(counts: Sequence[int], quantiles=(0.5, 0.9, 0.99)) -> Dict[str, float]:
    if not counts:
        return {"count": 0}
    xs = sorted(counts)
    out = {"count": len(xs), "mean": sum(xs) / len(xs), "min": xs[0], "max": xs[-1]}
    for q in quantiles:
        out[f"q{q:g}"] = xs[min(len(xs) - 1, int(q * (len(xs) - 1) + 0.5))]
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("data", type=Path)
    ap.add_argument("checkpoint_dir", type=Path)
    ap.add_argument("--field", action="append", default=None)
    a = ap.parse_args(argv)
    from keys_values_b200.tokenizer import Tokenizer

    tok = Tokenizer(a.checkpoint_dir)
    counts = token_counts(load_records(a.data), lambda s: tok.encode(s), a.field or ["instruction", "input", "output"])
    print(json.dumps(summarize(counts)))


if __name__ == "__main__":
    main()
