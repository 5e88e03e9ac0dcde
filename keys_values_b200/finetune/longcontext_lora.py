"""``finetune_long_lora``: long-context fine-tuning of LoRA adapters
(``keys_values/finetune/longcontext_lora.py:35-258``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, Optional, Union

from keys_values_b200.finetune import longcontext_full as full
from keys_values_b200.finetune.args import EvalArgs, GradientArgs, KVCacheArgs, LoRAArgs, OptimizerArgs, SDPAArgs, TrainArgs


def setup(checkpoint_dir: Union[str, Path], out_dir: Union[str, Path] = Path("out/finetune/long-lora"), lora: LoRAArgs = LoRAArgs(),
          yarn_rope: bool = True, **kwargs) -> None:
    full.setup(checkpoint_dir, out_dir, lora=lora, yarn_rope=yarn_rope, **kwargs)


full.inherit_cli_signature(setup, {'out_dir': Path('out/finetune/long-lora'), 'lora': LoRAArgs()})
