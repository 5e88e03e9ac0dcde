"""Sample-based metrics for generated answers (``keys_values/evaluation/metrics.py``):
exact / sub-exact match, ROUGE-n F1, NDCG@10 for rerank outputs, multiple-choice letter."""
from __future__ import annotations

import math
import re
import string
from collections import Counter
from typing import Dict, List, Sequence


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def exact_match(prediction: str, references: Sequence[str]) -> float:
    p = normalize_answer(prediction)
    return float(any(p == normalize_answer(r) for r in references))


def sub_exact_match(prediction: str, references: Sequence[str]) -> float:
    p = normalize_answer(prediction)
    return float(any(normalize_answer(r) in p for r in references if normalize_answer(r)))


def _ngrams(tokens: List[str], n: int) -> Counter:
    return Counter(tuple(tokens[i : i + n]) for i in range(len(tokens) - n + 1))


def rouge_n_f1(prediction: str, references: Sequence[str], n: int = 1) -> float:
    pt = normalize_answer(prediction).split()
    best = 0.0
    for r in references:
        rt = normalize_answer(r).split()
        pg, rg = _ngrams(pt, n), _ngrams(rt, n)
        overlap = sum((pg & rg).values())
        if overlap == 0:
            continue
        prec, rec = overlap / max(sum(pg.values()), 1), overlap / max(sum(rg.values()), 1)
        best = max(best, 2 * prec * rec / (prec + rec))
    return best


def ndcg_at_k(ranked_ids: Sequence[str], relevance: Dict[str, float], k: int = 10) -> float:
    dcg = sum(relevance.get(d, 0.0) / math.log2(i + 2) for i, d in enumerate(ranked_ids[:k]))
    ideal = sorted(relevance.values(), reverse=True)[:k]
    idcg = sum(r / math.log2(i + 2) for i, r in enumerate(ideal))
    return dcg / idcg if idcg > 0 else 0.0


def multiple_choice_letter(prediction: str, reference: str) -> float:
    m = re.search(r"correct answer is \(?([A-D])\)?", prediction) or re.search(r"\(([A-D])\)", prediction) or re.search(r"\b([A-D])\b", prediction)
    return float(m is not None and m.group(1) == reference.strip().strip("()"))


METRICS = {"exact_match": exact_match, "sub_exact_match": sub_exact_match, "rouge1_f1": lambda p, r: rouge_n_f1(p, r, 1),
           "rouge2_f1": lambda p, r: rouge_n_f1(p, r, 2)}
