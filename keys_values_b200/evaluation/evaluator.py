"""Generates answers for evaluation batches and scores them
(``keys_values/evaluation/evaluator.py:93-211``)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from keys_values_b200.evaluation.metrics import METRICS
from keys_values_b200.generate.base import batched_generate_fn


class SampleBasedMetricsEvaluator:
    def __init__(self, gpt_model, tokenizer, metric: str = "sub_exact_match", max_new_tokens: int = 64, prompt_chunksize: int = 1024,
                 parser: Optional[Callable[[str], str]] = None, sample_args: Optional[dict] = None):
        if metric not in METRICS:
            raise ValueError(f"metric = {metric} not supported; must be in {list(METRICS)}")
        self.gpt_model, self.tokenizer, self.metric_name, self.metric = gpt_model, tokenizer, metric, METRICS[metric]
        self.max_new_tokens, self.prompt_chunksize = max_new_tokens, prompt_chunksize
        self.parser = parser or str.strip  # the metrics strip lead-ins and quotes themselves
        self.sample_args = {k: v for k, v in (sample_args or dict(temperature=0.0)).items() if v is not None}

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


def split_prompts_and_references(batch: Dict[str, Any], tokenizer, pad_id: int = 0, ignore_index: int = -100):
    """Right-padded SFT batch (``input_ids``, ``labels`` masked on the prompt) → left-padded prompts
    ``(B, T_prompt)`` and, per row, the reference answer decoded from the unmasked labels."""
    ids, labels = batch["input_ids"], batch["labels"]
    B = ids.shape[0]
    is_target = labels != ignore_index
    first = torch.where(is_target.any(1), is_target.int().argmax(dim=1), torch.full((B,), ids.shape[1]))
    width = int(first.max())
    prompts = torch.full((B, width), pad_id, dtype=ids.dtype)
    refs: List[List[str]] = []
    eos = getattr(tokenizer, "eos_id", None)
    for b in range(B):
        n = int(first[b])
        prompts[b, width - n :] = ids[b, :n]
        ans = labels[b][is_target[b]]
        if eos is not None and ans.numel() and int(ans[-1]) == eos:
            ans = ans[:-1]
        refs.append([tokenizer.decode(ans)])
    return prompts, refs


def sample_metric_on_loader(gpt_model, tokenizer, loader, metric: str, device, max_batches: Optional[int] = None, max_new_tokens: int = 64,
                            prompt_chunksize: int = 1024, pad_id: int = 0, on_batch: Optional[Callable[[int, Dict[str, Any]], None]] = None) -> Dict[str, Any]:
    """Generate for up to ``max_batches`` batches of ``loader`` and average the metric.
    ``on_batch(batch_idx, result)`` sees every batch result (scores and generated texts)."""
    ev = SampleBasedMetricsEvaluator(gpt_model, tokenizer, metric, max_new_tokens, prompt_chunksize)
    scores: List[float] = []
    for k, batch in enumerate(loader):
        if max_batches is not None and k >= max_batches:
            break
        prompts, refs = split_prompts_and_references(batch, tokenizer, pad_id)
        gpt_model.reset()
        gpt_model.max_seq_length = prompts.shape[1] + max_new_tokens
        res = ev(prompts.to(device), refs)
        res["references"] = [r[0] for r in refs]
        scores.extend(res["scores"])
        if on_batch is not None:
            on_batch(k, res)
    return {"metric": metric, "mean": sum(scores) / max(len(scores), 1), "num_samples": len(scores)}
