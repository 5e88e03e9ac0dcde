"""Data modules that filter by token length and batch sequences of similar length
(``keys_values/data/module.py:107-457``), plus a synthetic source for benchmarks and tests."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import torch

from keys_values_b200.data.base import DataModule, SFTDataset, get_sft_collate_fn
from keys_values_b200.data.dataloader import MyDataLoader
from keys_values_b200.data.iterators import SimilarSequenceLengthSampler


class SequenceLengthFilteredDataModule(DataModule):
    """Wraps lists of SFT records: token lengths are taken from the records (``num_tokens_instruction``, filled by
    the dataset modules from their metadata files), from a JSON cache next to the data, or computed once; records
    longer than ``max_seq_length`` (or shorter than ``min_seq_length``) are dropped; batches are length-bucketed and
    rank-aware. With ``class_labels`` set the datasets are sequence-classification datasets (prompt + class index)."""

    def __init__(self, train_records: List[Dict[str, str]], val_records: List[Dict[str, str]], prompt_style=None, mask_prompt: bool = True,
                 min_seq_length: int = 0, max_seq_length: Optional[int] = None, seed: int = 42, num_workers: int = 0,
                 length_cache: Optional[Path] = None, longest_first: bool = False, shortest_first: bool = False, ignore_index: int = -100):
        if longest_first and shortest_first:
            raise ValueError("trainloader_longest_first and trainloader_shortest_first cannot both be set")
        self.train_records, self.val_records = train_records, val_records
        self.prompt_style, self.mask_prompt, self.ignore_index = prompt_style, mask_prompt, ignore_index
        self.min_seq_length, self.max_len_filter = min_seq_length, max_seq_length
        self.seed, self.num_workers, self.length_cache = seed, num_workers, length_cache
        self.longest_first, self.shortest_first = longest_first, shortest_first
        self.num_devices, self.rank = 1, 0
        self.tokenizer = None
        self.class_labels: Optional[Sequence[str]] = None
        self.train_dataset = self.val_dataset = None
        self._train_lengths: List[int] = []
        self._val_lengths: List[int] = []
        self._train_loader = None

    @property
    def model_name(self) -> str:
        """Name under which token lengths are filed: they depend on the tokenizer, i.e. on the model."""
        return str(getattr(self.tokenizer, "model_name", None) or "default")

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length: Optional[int] = None, num_devices: int = 1, rank: int = 0, **kwargs):
        super().connect(tokenizer, batch_size, max_seq_length)
        self.num_devices, self.rank = num_devices, rank
        if max_seq_length is not None and self.max_len_filter is None:
            self.max_len_filter = max_seq_length

    def _make_dataset(self, records):
        if self.class_labels is not None:
            from keys_values_b200.data.sequence_classification import SequenceClassificationDataset

            return SequenceClassificationDataset(records, self.tokenizer, self.prompt_style, self.class_labels)
        return SFTDataset(records, self.tokenizer, self.prompt_style, -1, self.mask_prompt, self.ignore_index)

    def _lengths(self, dataset, records, tag: str) -> List[int]:
        if records and all("num_tokens_instruction" in r for r in records):
            return [int(r["num_tokens_instruction"]) for r in records]
        if self.length_cache is not None:
            p = Path(self.length_cache) / f"lengths_{tag}.json"
            if p.is_file():
                cached = json.loads(p.read_text())
                if len(cached) == len(dataset):
                    return cached
        lengths = [int(dataset[i]["token_counts"]["raw"]) for i in range(len(dataset))]
        if self.length_cache is not None:
            Path(self.length_cache).mkdir(parents=True, exist_ok=True)
            (Path(self.length_cache) / f"lengths_{tag}.json").write_text(json.dumps(lengths))
        return lengths

    def _filter(self, records, tag, apply_limit: bool = True):
        lengths = self._lengths(self._make_dataset(records), records, tag)
        hi = self.max_len_filter if (apply_limit and self.max_len_filter is not None) else float("inf")
        keep = [i for i, n in enumerate(lengths) if self.min_seq_length <= n <= hi]
        return self._make_dataset([records[i] for i in keep]), [lengths[i] for i in keep]

    def setup(self, stage: str = "") -> None:
        self.train_dataset, self._train_lengths = self._filter(self.train_records, "train")
        self.val_dataset, self._val_lengths = self._filter(self.val_records, "val")

    def _loader(self, dataset, lengths, shuffle: bool):
        sampler = SimilarSequenceLengthSampler(lengths, self.batch_size, self.num_devices, self.rank, shuffle=shuffle,
                                               longest_first=self.longest_first and shuffle, seed=self.seed, drop_last=shuffle,
                                               shortest_first=self.shortest_first and shuffle)
        pad_id = getattr(self.tokenizer, "pad_id", None) or 0
        if self.class_labels is not None:
            from keys_values_b200.data.sequence_classification import get_seq_class_collate_fn

            collate = get_seq_class_collate_fn(pad_id=pad_id)
        else:
            collate = get_sft_collate_fn(pad_id=pad_id)
        return MyDataLoader(dataset, batch_sampler=sampler, num_workers=self.num_workers, collate_fn=collate)

    def train_dataloader(self):
        self._train_loader = self._loader(self.train_dataset, self._train_lengths, True)
        return self._train_loader

    def val_dataloader(self):
        return self._loader(self.val_dataset, self._val_lengths, False)

    def state_dict(self) -> Dict[str, Any]:
        return {"train_lengths": self._train_lengths, "val_lengths": self._val_lengths,
                "train_loader": self._train_loader.state_dict() if self._train_loader is not None else {}}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self._resume_loader_state = state.get("train_loader", {})


class _SyntheticDataset(torch.utils.data.Dataset):
    def __init__(self, n, seq_lengths, vocab_size, num_targets, seed):
        self.n, self.seq_lengths, self.vocab_size, self.num_targets, self.seed = n, seq_lengths, vocab_size, num_targets, seed

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed + idx)
        L = self.seq_lengths[idx % len(self.seq_lengths)]
        ids = torch.randint(0, self.vocab_size, (L + 1,), generator=g)
        labels = ids.clone()
        labels[: L + 1 - self.num_targets] = -100
        return {"input_ids": ids, "labels": labels, "token_counts": {"raw": L + 1, "raw_plus_prompt_template": L + 1}}


class SyntheticLongContext(DataModule):
    """Uniform random token sequences of given lengths with the loss on the final
    ``num_targets`` tokens: the data source of the benchmarks (no tokenizer, no network)."""

    def __init__(self, vocab_size: int, seq_lengths: Sequence[int] = (131072,), num_targets: int = 1024, num_train: int = 64, num_val: int = 8, seed: int = 0):
        self.vocab_size, self.seq_lengths, self.num_targets = vocab_size, list(seq_lengths), num_targets
        self.num_train, self.num_val, self.seed = num_train, num_val, seed
        self.num_devices, self.rank, self.batch_size = 1, 0, 1

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length=None, num_devices: int = 1, rank: int = 0, **kwargs):
        super().connect(tokenizer, batch_size, max_seq_length)
        self.num_devices, self.rank = num_devices, rank

    def _loader(self, n, seed, shuffle):
        ds = _SyntheticDataset(n, self.seq_lengths, self.vocab_size, self.num_targets, seed)
        lengths = [self.seq_lengths[i % len(self.seq_lengths)] + 1 for i in range(n)]
        sampler = SimilarSequenceLengthSampler(lengths, self.batch_size, self.num_devices, self.rank, shuffle=shuffle, seed=self.seed)
        return MyDataLoader(ds, batch_sampler=sampler, collate_fn=get_sft_collate_fn())

    def train_dataloader(self):
        return self._loader(self.num_train, self.seed, True)

    def val_dataloader(self):
        return self._loader(self.num_val, self.seed + 10_000, False)
