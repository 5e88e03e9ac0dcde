"""HELMET long-context benchmark tasks as supervised fine-tuning data (``keys_values/data/helmet.py:131-510``).

The development split of a task (built by :mod:`keys_values_b200.data.helmet_builder`) is divided into training
and validation data by ``val_split_fraction``; the evaluation split is the test set. Every instance carries its
fully formatted prompt, so no prompt style is applied. Token lengths per (task, context length, tokenizer, split)
are kept in ``metadata_dir/helmet_metadata.json``."""
from __future__ import annotations

import random
from typing import Any, Dict, List, Optional

from keys_values_b200.data.helmet_builder import DATASET_PARENT_DIR, LENGTHS, SUPPORTED_DATASET_KEYS, load_helmet_dev_eval
from keys_values_b200.data.metadata import LengthMetadata
from keys_values_b200.data.module import SequenceLengthFilteredDataModule

METADATA_FNAME = "helmet_metadata.json"
LENGTH_NAMES = {"8k": 8192, "16k": 16384, "32k": 32768, "64k": 65536, "128k": 131072}


def _as_text(output: Any) -> str:
    """Training target of an instance: the first of several gold answers."""
    if isinstance(output, (list, tuple)):
        return str(output[0]) if output else ""
    return str(output)


class Helmet(SequenceLengthFilteredDataModule):
    def __init__(self, dataset_key: str = "nq", max_length: str = "8k", dataset_parent_dir: str = DATASET_PARENT_DIR, mask_prompt: bool = True,
                 val_split_fraction: float = 0.1, ignore_index: int = -100, max_seq_length: Optional[int] = None, seed: int = 42,
                 metadata_dir: Optional[str] = None, trainloader_longest_first: bool = False, trainloader_shortest_first: bool = False,
                 recompute_lengths: bool = False, num_workers: int = 0, sources: Optional[Dict[str, List[Dict[str, Any]]]] = None):
        if dataset_key not in SUPPORTED_DATASET_KEYS:
            raise ValueError(f"dataset_key = {dataset_key} is not supported; choose from {SUPPORTED_DATASET_KEYS}")
        if max_length not in LENGTHS:
            raise ValueError(f"max_length = {max_length} must be one of {list(LENGTHS)}")
        if not 0.0 < val_split_fraction < 1.0:
            raise ValueError(f"val_split_fraction = {val_split_fraction} must lie in (0, 1)")
        super().__init__([], [], mask_prompt=mask_prompt, max_seq_length=max_seq_length, seed=seed, num_workers=num_workers,
                         longest_first=trainloader_longest_first, shortest_first=trainloader_shortest_first, ignore_index=ignore_index)
        self.dataset_key, self.max_length, self.dataset_parent_dir = dataset_key, max_length, dataset_parent_dir
        self.val_split_fraction, self.metadata_dir, self.recompute_lengths = val_split_fraction, metadata_dir, recompute_lengths
        self.test_records: List[Dict[str, Any]] = []
        self._sources = sources

    def _length_keys(self, split: str) -> List[str]:
        return [self.dataset_key, self.max_length, self.model_name, split]

    def prepare_data(self) -> None:
        processor = getattr(self.tokenizer, "processor", self.tokenizer)
        dev, evl = load_helmet_dev_eval(self.dataset_key, tokenizer=processor, max_length=self.max_length,
                                        dataset_parent_dir=self.dataset_parent_dir, sources=self._sources)
        meta = LengthMetadata(self.metadata_dir, METADATA_FNAME)
        splits = {}
        for split, data in (("dev", dev), ("eval", evl)):
            records = [{"instruction": r["input"], "output": _as_text(r["output"]), "query_id": r.get("query_id"), "all_outputs": r["output"]}
                       for r in data]
            lengths = None if self.recompute_lengths else meta.lengths(self._length_keys(split), len(records))
            if lengths is None and self.tokenizer is not None:
                lengths = [int(self.tokenizer.encode(r["instruction"]).numel()) for r in records]
                meta.store(self._length_keys(split), lengths)
            if lengths is not None:
                for r, n in zip(records, lengths):
                    r["num_tokens_instruction"] = n
            splits[split] = records
        dev_records = splits["dev"]
        order = list(range(len(dev_records)))
        random.Random(self.seed).shuffle(order)
        n_val = max(1, int(round(len(order) * self.val_split_fraction))) if order else 0
        self.val_records = [dev_records[i] for i in order[:n_val]]
        self.train_records = [dev_records[i] for i in order[n_val:]]
        self.test_records = splits["eval"]

    def setup(self, stage: str = "") -> None:
        if not self.train_records and not self.test_records:
            self.prepare_data()
        super().setup(stage)

    def test_dataloader(self):
        ds, lengths = self._filter(self.test_records, "test")
        return self._loader(ds, lengths, shuffle=False)

    @staticmethod
    def smart_lastrec_info():
        from keys_values_b200.kvcache.smart_lastrec import SmartInitialInformation

        return SmartInitialInformation(end_initial_regex=r"format:\nAnswer: \[answer\]\n", max_initial_fraction=0.1)
