"""Batches for evaluation runs that score several tasks (checkpoints × cache setups) on one dataset
(``keys_values/data/evaluation.py:25-230``).

Every rank iterates the same sequence of (task, batch) jobs — tasks in the outer loop, batches of
similar sequence length (shortest first) in the inner one — and claims jobs through lock files, so
faster ranks simply do more of them. With ``delay_tokenization`` a job is first returned as
``{task, orig_idx}`` only, so that jobs already done or locked are skipped without tokenizing.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterator, List, Sequence, Tuple

import torch

from keys_values_b200.data.constants import ORIG_IDX_NAME, TASK_NAME


class SimilarSequenceLengthWithTasksIterator:
    def __init__(self, sequence_lengths: Sequence[int], micro_batch_size: int, num_tasks: int):
        self.micro_batch_size, self.num_tasks = micro_batch_size, num_tasks
        self.num_batches = math.ceil(len(sequence_lengths) / micro_batch_size)
        self.dataset_size = self.num_batches * micro_batch_size
        order = torch.argsort(torch.tensor(list(sequence_lengths)), stable=True).tolist()
        # indexes >= len(sequence_lengths) are pad entries: they fill up the last (longest) batch
        self._permutation = order + list(range(len(sequence_lengths), self.dataset_size))
        self._pos = 0

    def __iter__(self):
        return self

    def __next__(self) -> Tuple[List[int], int]:
        if self._pos >= self.dataset_size * self.num_tasks:
            raise StopIteration
        task_idx, start = divmod(self._pos, self.dataset_size)
        self._pos += self.micro_batch_size
        return self._permutation[start : start + self.micro_batch_size], task_idx


class SimilarSequenceLengthWithTasksSampler:
    def __init__(self, sequence_lengths: Sequence[int], micro_batch_size: int, num_tasks: int):
        if micro_batch_size < 1 or num_tasks < 1 or len(sequence_lengths) == 0:
            raise ValueError("need micro_batch_size >= 1, num_tasks >= 1 and a non-empty dataset")
        self._kwargs = dict(sequence_lengths=list(sequence_lengths), micro_batch_size=micro_batch_size, num_tasks=num_tasks)
        self._len = math.ceil(len(sequence_lengths) / micro_batch_size) * num_tasks

    def __iter__(self) -> SimilarSequenceLengthWithTasksIterator:
        return SimilarSequenceLengthWithTasksIterator(**self._kwargs)

    def __len__(self) -> int:
        return self._len

    @property
    def batch_size(self) -> int:
        return self._kwargs["micro_batch_size"]

    @property
    def num_tasks(self) -> int:
        return self._kwargs["num_tasks"]


class EvaluationDataLoaderIterator:
    def __init__(self, dataset, batch_sampler: SimilarSequenceLengthWithTasksSampler, collate_fn: Callable[[List[Any]], Dict[str, Any]],
                 eval_tasks: List[str], delay_tokenization: bool):
        if len(eval_tasks) != batch_sampler.num_tasks:
            raise ValueError(f"len(eval_tasks) = {len(eval_tasks)} != {batch_sampler.num_tasks} = batch_sampler.num_tasks")
        self.dataset, self.collate_fn, self.eval_tasks, self.delay_tokenization = dataset, collate_fn, eval_tasks, delay_tokenization
        self._batch_iter = iter(batch_sampler)
        if len(dataset) != self._batch_iter.dataset_size:
            raise ValueError(f"len(dataset) = {len(dataset)} != {self._batch_iter.dataset_size} = batch_sampler.dataset_size")

    def __iter__(self):
        return self

    def __next__(self) -> Dict[str, Any]:
        inds, task_idx = next(self._batch_iter)
        job = {TASK_NAME: self.eval_tasks[task_idx], ORIG_IDX_NAME: inds}
        return job if self.delay_tokenization else self.fetch_full(job)

    def fetch_full(self, partial_batch: Dict[str, Any]) -> Dict[str, Any]:
        return {**partial_batch, **self.collate_fn([self.dataset[i] for i in partial_batch[ORIG_IDX_NAME]])}


class EvaluationDataLoader:
    def __init__(self, dataset, batch_sampler: SimilarSequenceLengthWithTasksSampler, collate_fn, eval_tasks: List[str],
                 delay_tokenization: bool = False):
        self._kwargs = dict(dataset=dataset, batch_sampler=batch_sampler, collate_fn=collate_fn, eval_tasks=eval_tasks,
                            delay_tokenization=delay_tokenization)

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        return EvaluationDataLoaderIterator(**self._kwargs)

    def __len__(self) -> int:
        return len(self._kwargs["batch_sampler"])

    @property
    def batch_size(self) -> int:
        return self._kwargs["batch_sampler"].batch_size

    @property
    def delay_tokenization(self) -> bool:
        return self._kwargs["delay_tokenization"]
