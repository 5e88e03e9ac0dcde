"""Datasets and collation for supervised fine-tuning on long sequences
(``keys_values/data/base.py:59-106``, ``sft_dataset.py:33-150``)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
from torch.utils.data import Dataset

IGNORE_INDEX = -100


class DataModule:
    """Interface of a data source: ``connect`` gets tokenizer and batch size, ``prepare_data``
    downloads/caches, ``setup`` builds the datasets, ``*_dataloader`` return loaders."""

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length: Optional[int] = None, **kwargs) -> None:
        self.tokenizer, self.batch_size, self.max_seq_length = tokenizer, batch_size, max_seq_length

    def prepare_data(self) -> None:
        pass

    def setup(self, stage: str = "") -> None:
        pass

    def train_dataloader(self):
        raise NotImplementedError

    def val_dataloader(self):
        raise NotImplementedError

    def state_dict(self) -> Dict[str, Any]:
        return {}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        pass


class SFTDataset(Dataset):
    """Records ``{"instruction": …, "output": …}`` → ``input_ids`` (prompt + response + eos) and
    ``labels`` (``-100`` on the prompt when ``mask_prompt``), with token counts."""

    def __init__(self, data: List[Dict[str, str]], tokenizer, prompt_style=None, max_seq_length: int = -1, mask_prompt: bool = True,
                 ignore_index: int = IGNORE_INDEX, transform: Optional[Callable[[Any], Any]] = None):
        self.data, self.tokenizer, self.prompt_style = data, tokenizer, prompt_style
        self.max_seq_length, self.mask_prompt, self.ignore_index, self.transform = max_seq_length, mask_prompt, ignore_index, transform

    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        ex = self.data[idx]
        if self.transform is not None:
            ex = self.transform(ex)
        prompt = ex["instruction"] if self.prompt_style is None else self.prompt_style.apply(prompt=ex["instruction"], **ex)
        enc_prompt = self.tokenizer.encode(prompt, max_length=self.max_seq_length)
        enc_resp = self.tokenizer.encode(ex["output"], bos=False, eos=True, max_length=self.max_seq_length)
        ids = torch.cat((enc_prompt, enc_resp)).to(torch.int64)
        if self.max_seq_length > 0:
            ids = ids[: self.max_seq_length]
        labels = ids.clone()
        if self.mask_prompt:
            labels[: len(enc_prompt)] = self.ignore_index
        return {"input_ids": ids, "labels": labels, "token_counts": {"raw": len(ids), "raw_plus_prompt_template": len(ids)}}


def pad_dataset(dataset: List[Any], multiple: int) -> List[Any]:
    """Repeat leading entries so that ``len(dataset)`` is a multiple of ``multiple``."""
    rem = len(dataset) % multiple
    if rem == 0 or not dataset:
        return dataset
    return list(dataset) + [dataset[i % len(dataset)] for i in range(multiple - rem)]


def common_collate_fn(samples: List[Dict[str, Any]], pad_id: int = 0, ignore_index: int = IGNORE_INDEX, max_seq_length: int = -1) -> Dict[str, Any]:
    """Right-pad ``input_ids`` (with ``pad_id``) and ``labels`` (with ``ignore_index``)."""
    batched: Dict[str, Any] = {}
    for key, fill in (("input_ids", pad_id), ("labels", ignore_index)):
        seqs = [s[key] for s in samples]
        if seqs[0].ndim == 0:
            batched[key] = torch.stack(seqs)
            continue
        batched[key] = torch.nn.utils.rnn.pad_sequence(seqs, batch_first=True, padding_value=fill)
        if max_seq_length > 0:
            batched[key] = batched[key][:, :max_seq_length]
    if "token_counts" in samples[0]:
        batched["token_counts"] = {k: torch.tensor([s["token_counts"][k] for s in samples], dtype=torch.int64) for k in samples[0]["token_counts"]}
    return batched


def get_sft_collate_fn(pad_id: int = 0, ignore_index: int = IGNORE_INDEX, max_seq_length: int = -1):
    from functools import partial

    return partial(common_collate_fn, pad_id=pad_id, ignore_index=ignore_index, max_seq_length=max_seq_length)
