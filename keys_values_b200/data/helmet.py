"""HELMET long-context benchmark tasks as SFT data (``keys_values/data/helmet.py:131-510``,
``load_helmet_dev_eval.py``).

The task files (JSON lines with ``context``/``question``/``answers``-style fields) must be
present under ``data_dir``: nothing is downloaded by this loader.
Records are turned into instruction/output pairs with the task's template and served through
:class:`SequenceLengthFilteredDataModule` (length filter by ``max_length`` such as ``64k``)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

from keys_values_b200.data.module import SequenceLengthFilteredDataModule

HELMET_TASKS = ("nq", "triviaqa", "hotpotqa", "popqa", "narrativeqa", "infbench_qa", "infbench_choice", "msmarco_rerank",
                "json_kv", "ruler_niah", "trec_coarse", "trec_fine", "banking77", "clinic150", "nlu")
LENGTH_NAMES = {"8k": 8192, "16k": 16384, "32k": 32768, "64k": 65536, "128k": 131072}

TEMPLATES = {
    "default": "Use the given documents to write a concise and short answer to the question. Write your answer in the following "
               "format:\nAnswer: [answer]\n\n{context}\n\nQuestion: {question}",
    "rerank": "You are provided with a list of documents, each indicated by their ID. Rank them by relevance to the query, most "
              "relevant first, as a list of IDs.\n\n{context}\n\nQuery: {question}",
    "icl": "Use the provided mapping from the text to label to assign a label to the text. Only output \"label: {{label}}\" and "
           "nothing else.\n\n{context}\n\n{question}",
}


def _template_for(task: str) -> str:
    if "rerank" in task:
        return TEMPLATES["rerank"]
    if task in ("trec_coarse", "trec_fine", "banking77", "clinic150", "nlu"):
        return TEMPLATES["icl"]
    return TEMPLATES["default"]


def load_helmet_records(data_dir: Path, task: str, max_length: str, split: str) -> List[Dict[str, str]]:
    if task not in HELMET_TASKS:
        raise ValueError(f"task = {task} not supported; must be in {HELMET_TASKS}")
    path = Path(data_dir) / task / f"{split}_{max_length}.jsonl"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: HELMET files must be placed there (no download in this environment)")
    template = _template_for(task)
    records = []
    with path.open() as fp:
        for line in fp:
            ex = json.loads(line)
            answers = ex.get("answers") or ex.get("answer") or ex.get("output") or ""
            answer = answers[0] if isinstance(answers, list) else answers
            records.append({"instruction": template.format(context=ex.get("context", ""), question=ex.get("question", ex.get("query", ""))),
                            "output": f"Answer: {answer}" if template is TEMPLATES["default"] else str(answer)})
    return records


class Helmet(SequenceLengthFilteredDataModule):
    def __init__(self, data_dir: Path = Path("data/helmet"), dataset_key: str = "nq", max_length: str = "64k", val_split_fraction: float = 0.1,
                 seed: int = 42, num_workers: int = 0, **kwargs):
        if max_length not in LENGTH_NAMES:
            raise ValueError(f"max_length = {max_length} must be one of {list(LENGTH_NAMES)}")
        self.data_dir, self.dataset_key, self.max_length_name = Path(data_dir), dataset_key, max_length
        self.val_split_fraction = val_split_fraction
        super().__init__([], [], max_seq_length=LENGTH_NAMES[max_length], seed=seed, num_workers=num_workers,
                         length_cache=self.data_dir / dataset_key / f"cache_{max_length}", **kwargs)

    def prepare_data(self) -> None:
        dev = load_helmet_records(self.data_dir, self.dataset_key, self.max_length_name, "dev")
        try:
            val = load_helmet_records(self.data_dir, self.dataset_key, self.max_length_name, "eval")
        except FileNotFoundError:
            n_val = max(1, int(len(dev) * self.val_split_fraction))
            dev, val = dev[n_val:], dev[:n_val]
        self.train_records, self.val_records = dev, val

    def setup(self, stage: str = "") -> None:
        if not self.train_records:
            self.prepare_data()
        super().setup(stage)

    @staticmethod
    def smart_lastrec_info():
        from keys_values_b200.kvcache.smart_lastrec import SmartInitialInformation

        return SmartInitialInformation(end_initial_regex=r"format:\nAnswer: \[answer\]\n", max_initial_fraction=0.1)
