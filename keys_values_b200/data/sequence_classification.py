"""In-memory dataset for fine-tuning a sequence-classification head
(``keys_values/data/sequence_classification.py:32-150``)."""
from __future__ import annotations

from functools import partial
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
from torch.utils.data import Dataset

from keys_values_b200.data.constants import INPUT_IDS_NAME, LABELS_NAME, POSITION_NAME, is_pad_datacase


class SequenceClassificationDataset(Dataset):
    """Records ``{"instruction": …, "output": <one of class_labels>}`` → prompt token ids (``eos``
    appended) and the index of the label. Pad records may only stand at the end."""

    def __init__(self, data: List[Dict[str, Any]], tokenizer, prompt_style, class_labels: Iterable[str],
                 max_seq_length: Optional[int] = None, transform: Optional[Callable[[Dict[str, Any]], Dict[str, Any]]] = None):
        self.data, self.tokenizer, self.prompt_style = data, tokenizer, prompt_style
        self.max_seq_length, self.transform = max_seq_length, transform
        self.class_labels = tuple(class_labels)
        if len(set(self.class_labels)) != len(self.class_labels):
            raise ValueError(f"class_labels = {self.class_labels}, must not have duplicate entries")
        index = {label: i for i, label in enumerate(self.class_labels)}
        self._label_indexes: List[Optional[int]] = []
        in_padding = False
        for idx, example in enumerate(data):
            if is_pad_datacase(example):
                in_padding = True
                self._label_indexes.append(None)
                continue
            if in_padding:
                raise ValueError(f"data can only contain pad entries at the end, but entry {idx} is not padding")
            if example["output"] not in index:
                raise ValueError(f"data[{idx}]['output'] = '{example['output']}' invalid, must lie in {self.class_labels}")
            self._label_indexes.append(index[example["output"]])

    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        if not 0 <= idx < len(self.data):
            raise IndexError(f"index {idx} out of range, must be in [0, {len(self.data)})")
        example, label = self.data[idx], self._label_indexes[idx]
        if label is None:
            return example
        if self.transform is not None:
            example = self.transform(example)
        prompt = example["instruction"] if self.prompt_style is None else self.prompt_style.apply(prompt=example["instruction"], **example)
        ids = self.tokenizer.encode(prompt, bos=False, eos=True, max_length=-1 if self.max_seq_length is None else self.max_seq_length)
        counts = {"raw_plus_prompt_template": len(ids)}
        raw = example.get("num_tokens_instruction")
        if raw is None and self.transform is None and self.prompt_style is None:
            raw = len(ids)
        if raw is not None:
            counts["raw"] = raw
        out = {INPUT_IDS_NAME: ids.to(torch.int64), LABELS_NAME: label, "token_counts": counts}
        if POSITION_NAME in example:
            out[POSITION_NAME] = example[POSITION_NAME]
        return out


def _seq_class_collate_fn(samples: List[Dict[str, Any]], pad_id: int = 0) -> Dict[str, Any]:
    samples = [s for s in samples if not is_pad_datacase(s)]
    ids = torch.nn.utils.rnn.pad_sequence([s[INPUT_IDS_NAME] for s in samples], batch_first=True, padding_value=pad_id)
    batch: Dict[str, Any] = {INPUT_IDS_NAME: ids, LABELS_NAME: torch.tensor([s[LABELS_NAME] for s in samples], dtype=torch.int64)}
    keys = set.intersection(*(set(s["token_counts"]) for s in samples))
    batch["token_counts"] = {k: torch.tensor([s["token_counts"][k] for s in samples], dtype=torch.int64) for k in sorted(keys)}
    return batch


def get_seq_class_collate_fn(pad_id: int = 0):
    return partial(_seq_class_collate_fn, pad_id=pad_id)
