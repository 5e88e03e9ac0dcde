"""Sample-based metrics for generated answers (``keys_values/evaluation/metrics.py``): exact and sub-exact match
(optionally fuzzy), ROUGE-n F1, NDCG@10 over ranked id lists, the multiple-choice letter and the recalled value of
the synthetic tasks."""
from __future__ import annotations

import math
import re
import string
from collections import Counter
from decimal import Decimal, InvalidOperation
from difflib import SequenceMatcher
from typing import Dict, Iterable, List, Optional, Sequence, Union

from keys_values_b200.evaluation.response_parser import extract_choice_letter, extract_value_token, normalize_string_response

Target = Union[str, int, float]


def normalize_answer(s: str) -> str:
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    return " ".join(re.sub(r"\b(a|an|the)\b", " ", s).split())


def _as_list(references) -> List[str]:
    if isinstance(references, (list, tuple)):
        return [str(r) for r in references]
    return [str(references)]


def _word_tokens(s: str) -> List[str]:
    return re.sub(r"[^\w\s]", " ", s.lower()).split()


def sub_exact_similarity(a: str, b: str) -> float:
    """Order-insensitive similarity in [0, 1]: the larger of the Jaccard index of the two token multisets and the
    character similarity of the sorted token strings (which forgives small typos)."""
    ta, tb = _word_tokens(a), _word_tokens(b)
    ca, cb = Counter(ta), Counter(tb)
    union = sum((ca | cb).values())
    jaccard = sum((ca & cb).values()) / union if union else 0.0
    sa, sb = " ".join(sorted(ta)), " ".join(sorted(tb))
    chars = SequenceMatcher(None, sa, sb).ratio() if (sa or sb) else 0.0
    return max(jaccard, chars)


def exact_match(prediction: str, references) -> float:
    """1 if the reply, stripped of lead-ins and quotes, equals one of the references (also after lower-casing and
    dropping punctuation and articles)."""
    raw = normalize_string_response(prediction)
    p = normalize_answer(raw)
    return float(any(raw == r or p == normalize_answer(r) for r in _as_list(references)))


def sub_exact_match(prediction: str, references, threshold: Optional[float] = None) -> float:
    """1 if a reference occurs in the reply (case-insensitive, after stripping lead-ins); with ``threshold`` also if
    :func:`sub_exact_similarity` reaches it."""
    raw = normalize_string_response(prediction).lower()
    p = normalize_answer(raw)
    for r in _as_list(references):
        rl, rn = r.lower(), normalize_answer(r)
        if (rl and rl in raw) or (rn and rn in p):
            return 1.0
        if threshold is not None and sub_exact_similarity(raw, rl) >= threshold:
            return 1.0
    return 0.0


def _ngrams(tokens: List[str], n: int) -> Counter:
    return Counter(tuple(tokens[i : i + n]) for i in range(len(tokens) - n + 1))


def rouge_n_f1(prediction: str, references, n: int = 1) -> float:
    pt = normalize_answer(prediction).split()
    best = 0.0
    for r in _as_list(references):
        pg, rg = _ngrams(pt, n), _ngrams(normalize_answer(r).split(), n)
        overlap = sum((pg & rg).values())
        if overlap:
            prec, rec = overlap / max(sum(pg.values()), 1), overlap / max(sum(rg.values()), 1)
            best = max(best, 2 * prec * rec / (prec + rec))
    return best


def ndcg_at_k(ranked_ids: Sequence[str], relevance: Dict[str, float], k: int = 10) -> float:
    """NDCG@k with graded relevance per document id (linear gain)."""
    dcg = sum(relevance.get(d, 0.0) / math.log2(i + 2) for i, d in enumerate(ranked_ids[:k]))
    ideal = sorted(relevance.values(), reverse=True)[:k]
    idcg = sum(r / math.log2(i + 2) for i, r in enumerate(ideal))
    return dcg / idcg if idcg > 0 else 0.0


def _canonical_number(x) -> Optional[str]:
    try:
        d = Decimal(str(x).strip())
    except (InvalidOperation, ValueError):
        return None
    d = Decimal(0) if d == 0 else d
    s = format(d.normalize(), "f")
    s = s.rstrip("0").rstrip(".") if "." in s else s
    return s or "0"


def ndcg_at_10_ranked_numbers(pred: Iterable[str], target: Iterable[str], *, k: int = 10) -> float:
    """NDCG@k of a predicted ranking of numeric ids against the ideal ranking ``target``: the id at target rank
    ``i < k`` has relevance ``k − i`` (exponential gain ``2^rel − 1``), ids are compared as numbers ("07" = "7.0"),
    and a repeated prediction is credited once."""
    ideal: List[str] = []
    for t in target:
        c = _canonical_number(t)
        if c is not None and c not in ideal:
            ideal.append(c)
    if not ideal or k <= 0:
        return 0.0
    rel = {v: float(k - i) for i, v in enumerate(ideal[:k])}
    gains, seen = [], set()
    for p in [c for c in (_canonical_number(x) for x in pred) if c is not None][:k]:
        gains.append(rel[p] if p in rel and p not in seen else 0.0)
        seen.add(p)
    dcg = sum((2.0**g - 1.0) / math.log2(i + 2) for i, g in enumerate(gains))
    idcg = sum((2.0 ** float(k - i) - 1.0) / math.log2(i + 2) for i in range(min(k, len(ideal))))
    return dcg / idcg if idcg else 0.0


def multiple_choice_letter(prediction: str, reference: str, choices: str = "ABCD") -> float:
    want = str(reference).strip().strip("()").upper()[:1]
    return float(bool(want) and extract_choice_letter(normalize_string_response(prediction), choices=choices) == want)


def synthetic_value_match(prediction: str, references) -> float:
    """Recall tasks (needle / JSON key-value): the value token of the reply equals one of the references, or every
    reference occurs in the reply (tasks that ask for several values)."""
    refs = _as_list(references)
    token = extract_value_token(prediction)
    if token and any(token == r.strip() for r in refs):
        return 1.0
    low = prediction.lower()
    return float(bool(refs) and all(r.strip().lower() in low for r in refs))


METRICS = {"exact_match": exact_match, "sub_exact_match": sub_exact_match, "rouge1_f1": lambda p, r: rouge_n_f1(p, r, 1),
           "rouge2_f1": lambda p, r: rouge_n_f1(p, r, 2), "multiple_choice": lambda p, r: multiple_choice_letter(p, _as_list(r)[0]),
           "synthetic_value": synthetic_value_match,
           "ndcg_at_10": lambda p, r: ndcg_at_10_ranked_numbers(re.findall(r"\d+", p), re.findall(r"\d+", " ".join(_as_list(r))))}

# metric that goes with a HELMET task (SampleBasedMetricsEvaluator.metric_for_helmet_task in the reference)
HELMET_TASK_METRIC = {
    **{k: "sub_exact_match" for k in ("nq", "trivia_qa", "hotpot_qa", "pop_qa", "json_kv")},
    **{k: "exact_match" for k in ("trec_coarse", "trec_fine", "nlu", "banking77", "clinc150", "infinite_bench_mc")},
    **{k: "synthetic_value" for k in ("ruler_mk_needle", "ruler_mk_uuid", "ruler_mv")},
    **{k: "rouge1_f1" for k in ("narrative_qa", "infinite_bench_qa", "infinite_bench_sum", "multi_lex_sum", "alce_asqa", "alce_qampari")},
    "ms_macro": "ndcg_at_10",
}
