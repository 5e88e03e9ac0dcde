"""Generates answers for evaluation batches and scores them
(``keys_values/evaluation/evaluator.py:93-211``)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from keys_values_b200.evaluation.metrics import METRICS
from keys_values_b200.evaluation.response_parser import parse_answer
from keys_values_b200.generate.base import batched_generate_fn


class SampleBasedMetricsEvaluator:
    def __init__(self, gpt_model, tokenizer, metric: str = "sub_exact_match", max_new_tokens: int = 64, prompt_chunksize: int = 1024,
                 parser: Callable[[str], str] = parse_answer, sample_args: Optional[dict] = None):
        if metric not in METRICS:
            raise ValueError(f"metric = {metric} not supported; must be in {list(METRICS)}")
        self.gpt_model, self.tokenizer, self.metric_name, self.metric = gpt_model, tokenizer, metric, METRICS[metric]
        self.max_new_tokens, self.prompt_chunksize, self.parser = max_new_tokens, prompt_chunksize, parser
        self.sample_args = sample_args or dict(temperature=0.0)

    @torch.no_grad()
    def __call__(self, prompts: torch.Tensor, references: Sequence[Sequence[str]]) -> Dict[str, Any]:
        """``prompts (B, T)`` left-padded token ids; ``references``: accepted answers per row."""
        B, T = prompts.shape
        stop = ([self.tokenizer.eos_id],) if getattr(self.tokenizer, "eos_id", None) is not None else ()
        rows: List[List[int]] = [[] for _ in range(B)]
        for toks in batched_generate_fn(self.gpt_model, prompts, T + self.max_new_tokens, self.prompt_chunksize, self.sample_args, stop,
                                        include_prompt=False, include_eos=False):
            for b, t in enumerate(toks):
                if t is not None:
                    rows[b].append(int(t))
        texts = [self.tokenizer.decode(r) for r in rows]
        scores = [self.metric(self.parser(t), refs) for t, refs in zip(texts, references)]
        return {"metric": self.metric_name, "scores": scores, "mean": sum(scores) / max(len(scores), 1), "generated": texts}
