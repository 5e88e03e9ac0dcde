"""LongBench-v2 multiple-choice tasks as SFT data (``keys_values/data/longbench_v2.py:65-640``).
The JSON file must be available locally (``data_dir/data.json``); nothing is downloaded."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

from keys_values_b200.data.module import SequenceLengthFilteredDataModule

TEMPLATE = ("Please read the following text and answer the question below.\n\n<text>\n{context}\n</text>\n\nWhat is the correct "
            "answer to this question: {question}\nChoices:\n(A) {choice_A}\n(B) {choice_B}\n(C) {choice_C}\n(D) {choice_D}\n\n"
            "Format your response as follows: \"The correct answer is (insert answer here)\".")


def load_longbench_records(path: Path, truncate_context_chars: Optional[int] = None) -> List[Dict[str, str]]:
    if not Path(path).is_file():
        raise FileNotFoundError(f"{path} not found: LongBench-v2 data must be placed there (no download in this environment)")
    data = json.loads(Path(path).read_text())
    records = []
    for ex in data:
        ctx = ex["context"]
        if truncate_context_chars is not None and len(ctx) > truncate_context_chars:
            half = truncate_context_chars // 2
            ctx = ctx[:half] + ctx[-half:]
        records.append({"instruction": TEMPLATE.format(context=ctx, question=ex["question"], choice_A=ex["choice_A"], choice_B=ex["choice_B"],
                                                       choice_C=ex["choice_C"], choice_D=ex["choice_D"]),
                        "output": f"The correct answer is ({ex['answer']})"})
    return records


class LongBenchV2(SequenceLengthFilteredDataModule):
    def __init__(self, data_dir: Path = Path("data/longbench_v2"), val_split_fraction: float = 0.1, max_seq_length: Optional[int] = None,
                 truncate_context_chars: Optional[int] = None, seed: int = 42, **kwargs):
        self.data_dir, self.val_split_fraction, self.truncate_context_chars = Path(data_dir), val_split_fraction, truncate_context_chars
        super().__init__([], [], max_seq_length=max_seq_length, seed=seed, length_cache=self.data_dir / "cache", **kwargs)

    def prepare_data(self) -> None:
        recs = load_longbench_records(self.data_dir / "data.json", self.truncate_context_chars)
        n_val = max(1, int(len(recs) * self.val_split_fraction))
        self.train_records, self.val_records = recs[n_val:], recs[:n_val]

    def setup(self, stage: str = "") -> None:
        if not self.train_records:
            self.prepare_data()
        super().setup(stage)

    @staticmethod
    def smart_lastrec_info():
        from keys_values_b200.kvcache.smart_lastrec import SmartInitialInformation

        return SmartInitialInformation(end_initial_regex=r"<text>\n", max_initial_fraction=0.05)


class LongBenchV2Truncated(LongBenchV2):
    """Contexts cut in the middle to at most ``truncate_context_chars`` characters."""

    def __init__(self, truncate_context_chars: int = 400_000, **kwargs):
        super().__init__(truncate_context_chars=truncate_context_chars, **kwargs)
