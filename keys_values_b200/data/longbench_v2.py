"""LongBench-v2 multiple-choice tasks as fine-tuning data (``keys_values/data/longbench_v2.py:65-640``).

Records come from ``datasets.load_dataset(repo_id)`` (a hub id or a local directory with the data files), are
turned into the benchmark's zero-shot prompt, filtered to prompts of at most ``max_seq_length`` tokens, and
served for next-token prediction (the answer letter follows "The correct answer is ") or, with a
sequence-classification head, as prompts with a class index. Token lengths per tokenizer are kept in
``metadata_dir/longbench_v2_metadata.json``; ``test_set_tag="rest"`` keeps the records that are too long for
training as a test set, shortest first."""
from __future__ import annotations

import os
import random
from typing import Any, Dict, List, Optional, Tuple

from keys_values_b200.data.metadata import LengthMetadata
from keys_values_b200.data.module import SequenceLengthFilteredDataModule

METADATA_FNAME = "longbench_v2_metadata.json"
CLASS_LABELS = ("A", "B", "C", "D")
SUPPORTED_TEST_SET_TAGS = ("rest",)
NEXT_TOKEN_HEAD = "next_token_prediction"
SUPPORTED_HEAD_MODELS = (NEXT_TOKEN_HEAD, "seq_classification_on_logits", "seq_classification")

PROMPT_HEAD = "Please read the following text and answer the question below.\n\n<text>\n"
PROMPT_TAIL = ("\n</text>\n\nWhat is the correct answer to this question: {question}\nChoices:\nA: {choice_A}\nB: {choice_B}\nC: {choice_C}\n"
               "D: {choice_D}\n\n")
PROMPT_FINAL = {
    NEXT_TOKEN_HEAD: 'Format your response as follows: "The correct answer is (insert answer here)".\n\nAnswer:\nThe correct answer is ',
    "seq_classification_on_logits": "The correct answer is ",
    "seq_classification": "The correct answer is ",
}


def get_instruction_template(head_model: str) -> Tuple[str, Tuple[str, ...]]:
    return PROMPT_HEAD + "{context}" + PROMPT_TAIL + PROMPT_FINAL[head_model], ("context", "question", "choice_A", "choice_B", "choice_C", "choice_D")


def format_record(entry: Dict[str, Any], head_model: str, context: Optional[str] = None) -> Dict[str, Any]:
    fields = {k: entry[k] for k in ("question", "choice_A", "choice_B", "choice_C", "choice_D")}
    ctx = entry["context"] if context is None else context
    return {"instruction": PROMPT_HEAD + ctx + PROMPT_TAIL.format(**fields) + PROMPT_FINAL[head_model], "output": entry["answer"]}


def truncated_context(entry: Dict[str, Any], tokenizer, head_model: str, width: int) -> str:
    """Tail of the context such that the whole prompt has at most ``width`` tokens (the head of a long document goes)."""
    fields = {k: entry[k] for k in ("question", "choice_A", "choice_B", "choice_C", "choice_D")}
    fixed = tokenizer.encode(PROMPT_HEAD).numel() + tokenizer.encode(PROMPT_TAIL.format(**fields) + PROMPT_FINAL[head_model]).numel()
    room = width - fixed
    if room <= 0:
        raise ValueError(f"truncation_context_width = {width} leaves no room for the context ({fixed} tokens of question and choices)")
    ids = tokenizer.encode(entry["context"])
    if ids.numel() <= room:
        return entry["context"]
    return entry["context"][-len(tokenizer.decode(ids[-room:])):]


class LongBenchV2(SequenceLengthFilteredDataModule):
    def __init__(self, mask_prompt: bool = True, val_split_fraction: float = 0.1, ignore_index: int = -100, max_seq_length: Optional[int] = 100000,
                 seed: int = 42, repo_id: str = "THUDM/LongBench-v2", access_token: Optional[str] = None, metadata_dir: Optional[str] = None,
                 debug_num_cases: Optional[int] = None, trainloader_longest_first: bool = False, trainloader_shortest_first: bool = False,
                 test_set_tag: Optional[str] = None, recompute_lengths: bool = False, num_workers: int = 0):
        if test_set_tag is not None and test_set_tag not in SUPPORTED_TEST_SET_TAGS:
            raise ValueError(f"test_set_tag = {test_set_tag} is not supported, must be None or in {SUPPORTED_TEST_SET_TAGS}")
        super().__init__([], [], mask_prompt=mask_prompt, max_seq_length=max_seq_length, seed=seed, num_workers=num_workers,
                         longest_first=trainloader_longest_first, shortest_first=trainloader_shortest_first, ignore_index=ignore_index)
        self.val_split_fraction, self.repo_id, self.metadata_dir = val_split_fraction, repo_id, metadata_dir
        self.access_token = os.getenv("HF_TOKEN") if access_token is None else access_token
        self.debug_num_cases, self.test_set_tag, self.recompute_lengths = debug_num_cases, test_set_tag, recompute_lengths
        self.head_model = NEXT_TOKEN_HEAD
        self.test_records: List[Dict[str, Any]] = []

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length: Optional[int] = None, num_devices: int = 1, rank: int = 0, **kwargs):
        super().connect(tokenizer, batch_size, max_seq_length, num_devices, rank, **kwargs)
        head = kwargs.get("head_model", NEXT_TOKEN_HEAD)
        if head not in SUPPORTED_HEAD_MODELS:
            raise ValueError(f"head_model '{head}' not supported, must be in {SUPPORTED_HEAD_MODELS}")
        self.head_model = head
        self.class_labels = None if head == NEXT_TOKEN_HEAD else CLASS_LABELS

    def _raw(self):
        from datasets import load_dataset

        return load_dataset(self.repo_id, token=self.access_token)["train"]

    def _context_for(self, idx: int, entry: Dict[str, Any]) -> Optional[str]:
        return None  # the full context; the truncated variant overrides this

    def prepare_data(self) -> None:
        data = self._raw()
        meta = LengthMetadata(self.metadata_dir, METADATA_FNAME)
        lengths = None if self.recompute_lengths else meta.lengths([self.model_name], len(data))
        computed: List[int] = []
        kept: List[Dict[str, Any]] = []
        rest: List[Dict[str, Any]] = []
        limit = self.max_len_filter
        for idx, entry in enumerate(data):
            rec = format_record(entry, self.head_model, self._context_for(idx, entry))
            if lengths is not None:
                n = lengths[idx]
            else:
                n = int(self.tokenizer.encode(format_record(entry, self.head_model)["instruction"]).numel())
                computed.append(n)
            rec["num_tokens_instruction"] = n
            if limit is None or n <= limit:
                if self.debug_num_cases is None or len(kept) < self.debug_num_cases:
                    kept.append(rec)
            elif self.test_set_tag == "rest":
                rest.append(rec)
        if lengths is None:
            meta.store([self.model_name], computed)
        order = list(range(len(kept)))
        random.Random(self.seed).shuffle(order)
        n_val = max(1, int(round(len(order) * self.val_split_fraction))) if order else 0
        self.val_records = [kept[i] for i in order[:n_val]]
        self.train_records = [kept[i] for i in order[n_val:]]
        self.test_records = sorted(rest, key=lambda r: r["num_tokens_instruction"])

    def setup(self, stage: str = "") -> None:
        if not self.train_records:
            self.prepare_data()
        super().setup(stage)

    def test_dataloader(self):
        if not self.test_records:
            return None
        ds, lengths = self._filter(self.test_records, "test", apply_limit=False)
        return self._loader(ds, lengths, shuffle=False)

    def head_model_kwargs(self, name: str, tokenizer=None) -> Dict[str, Any]:
        """Constructor arguments of head ``name`` for this dataset (class-label tokens need the tokenizer)."""
        if name == NEXT_TOKEN_HEAD:
            return {}
        if name == "seq_classification":
            return {"num_classes": len(CLASS_LABELS)}
        tokenizer = tokenizer or self.tokenizer
        if tokenizer is None:
            raise IndexError("the class-label tokens need a tokenizer: pass one or call connect first")
        tokens = []
        for label in CLASS_LABELS:
            ids = tokenizer.encode(label, bos=False)
            if ids.numel() != 1:
                raise ValueError(f"class label {label} maps to tokens {ids.tolist()}, but must map to a single token")
            tokens.append(int(ids.item()))
        return {"class_label_tokens": tokens}

    @staticmethod
    def smart_lastrec_info():
        from keys_values_b200.kvcache.smart_lastrec import SmartInitialInformation

        return SmartInitialInformation(end_initial_regex=r"<text>\n", max_initial_fraction=0.1)


class LongBenchV2Truncated(LongBenchV2):
    """The baseline that long-context fine-tuning is compared with: the same records, with the head of the context
    cut so that a prompt has at most ``truncation_context_width`` tokens. Needs the length metadata written by
    :class:`LongBenchV2` (records are selected by their untruncated length)."""

    def __init__(self, metadata_dir: Optional[str] = None, truncation_context_width: Optional[int] = None, **kwargs):
        if metadata_dir is None:
            raise ValueError("metadata_dir must be given and hold the metadata file: use LongBenchV2 first to create it")
        super().__init__(metadata_dir=metadata_dir, **kwargs)
        self.truncation_context_width = truncation_context_width

    def connect(self, tokenizer=None, batch_size: int = 1, max_seq_length: Optional[int] = None, num_devices: int = 1, rank: int = 0, **kwargs):
        super().connect(tokenizer, batch_size, max_seq_length, num_devices, rank, **kwargs)
        self.truncation_context_width = kwargs.get("truncation_context_width", self.truncation_context_width)
        if self.truncation_context_width is None:
            raise ValueError("truncation_context_width must be provided")

    def prepare_data(self) -> None:
        if LengthMetadata(self.metadata_dir, METADATA_FNAME).lengths([self.model_name]) is None:
            raise FileNotFoundError(f"no token lengths for '{self.model_name}' in {self.metadata_dir}/{METADATA_FNAME}: use LongBenchV2 first")
        super().prepare_data()

    def _context_for(self, idx: int, entry: Dict[str, Any]) -> Optional[str]:
        return truncated_context(entry, self.tokenizer, self.head_model, self.truncation_context_width)
