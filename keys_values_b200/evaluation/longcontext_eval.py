"""``eval_long``: evaluation of one fine-tuning output directory with the settings it was
trained with (``keys_values/evaluation/longcontext_eval.py:22-165``); a thin front end of
:mod:`keys_values_b200.evaluation.longcontext_eval_ext`."""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Union

from keys_values_b200.evaluation import longcontext_eval_ext as ext
from keys_values_b200.finetune.args import EvalArgs


def setup(out_dir: Union[str, Path], data=None, eval: EvalArgs = EvalArgs(), devices: int = 1, precision: Optional[str] = None,
          checkpoints: Optional[List[str]] = None, batch_size: int = 1) -> None:
    ext.setup(out_dir, checkpoints=checkpoints, data=data, eval=eval, devices=devices, precision=precision, batch_size=batch_size)
