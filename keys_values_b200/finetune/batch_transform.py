"""Batch transforms: right-padded ``(input_ids, labels)`` → left-padded prompts + targets.

All rows of a batch must share the same prompt/target split, because the chunked
forward computes the loss on the last ``targets.shape[1]`` positions. Rows are therefore
re-aligned so that their prompts end at the same position (left padding), and
``input_ids = tokens[:, :-1]``, ``targets = labels[:, max_prompt_len:]``.
Parity: ``keys_values/finetune/batch_transform.py:52-255``.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

IGNORE_INDEX = -100


class BatchTransform:
    def __call__(self, batch: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        raise NotImplementedError


class SFTBatchTransform(BatchTransform):
    def __init__(self, pad_id: int = 0, ignore_index: int = IGNORE_INDEX, eos_id: Optional[int] = None):
        self.pad_id, self.ignore_index, self.eos_id = pad_id, ignore_index, eos_id

    def __call__(self, batch):
        ids, labels = batch["input_ids"], batch["labels"]
        B, T = ids.shape
        is_target = labels != self.ignore_index
        seq_len = batch.get("token_counts", {}).get("raw") if isinstance(batch.get("token_counts"), dict) else None
        if seq_len is None:
            # length of a row = index of the last non-pad token + 1 (targets are never padding)
            nonpad = (ids != self.pad_id) | is_target
            seq_len = T - nonpad.flip(1).int().argmax(dim=1)
        else:
            seq_len = seq_len.view(-1)
        first_target = torch.where(is_target.any(1), is_target.int().argmax(dim=1), seq_len)
        prompt_len = first_target
        target_len = seq_len - first_target
        max_prompt, max_target = int(prompt_len.max()), int(target_len.max())
        total = max_prompt + max_target
        new_ids = torch.full((B, total), self.pad_id, dtype=ids.dtype, device=ids.device)
        new_labels = torch.full((B, total), self.ignore_index, dtype=labels.dtype, device=labels.device)
        for b in range(B):
            pl, tl = int(prompt_len[b]), int(target_len[b])
            new_ids[b, max_prompt - pl : max_prompt + tl] = ids[b, : pl + tl]
            new_labels[b, max_prompt : max_prompt + tl] = labels[b, pl : pl + tl]
        # model input is tokens[:-1]; position t predicts token t+1
        return {"input_ids": new_ids[:, :-1].contiguous(), "targets": new_labels[:, max_prompt:].contiguous()}


class SequenceClassificationBatchTransform(BatchTransform):
    """``labels`` is one class index per row; inputs are left-padded to equal length."""

    def __init__(self, pad_id: int = 0):
        self.pad_id = pad_id

    def __call__(self, batch):
        ids, labels = batch["input_ids"], batch["labels"]
        B, T = ids.shape
        nonpad = ids != self.pad_id
        seq_len = T - nonpad.flip(1).int().argmax(dim=1)
        max_len = int(seq_len.max())
        new_ids = torch.full((B, max_len), self.pad_id, dtype=ids.dtype, device=ids.device)
        for b in range(B):
            n = int(seq_len[b])
            new_ids[b, max_len - n :] = ids[b, :n]
        return {"input_ids": new_ids, "targets": labels.view(B, 1)}


class BatchTransformFactory:
    @staticmethod
    def from_head_model(head_model_name: str, pad_id: int = 0, eos_id: Optional[int] = None, **kwargs) -> BatchTransform:
        from keys_values_b200.models.head_model import CrossEntropyOnLogits

        if head_model_name == CrossEntropyOnLogits.NAME:
            return SFTBatchTransform(pad_id=pad_id, eos_id=eos_id, **kwargs)
        return SequenceClassificationBatchTransform(pad_id=pad_id)
