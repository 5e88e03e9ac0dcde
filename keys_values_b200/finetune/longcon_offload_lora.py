"""``finetune_offload_lora``: LoRA fine-tuning with host-resident checkpoints and optimizer state
(``keys_values/finetune/longcon_offload_lora.py``; see :mod:`keys_values_b200.finetune.longcon_offload_full`)."""
from __future__ import annotations

from pathlib import Path
from typing import Union

from keys_values_b200.finetune import longcontext_full as full
from keys_values_b200.finetune.args import LoRAArgs


def setup(checkpoint_dir: Union[str, Path], out_dir: Union[str, Path] = Path("out/finetune/offload-lora"), lora: LoRAArgs = LoRAArgs(), **kwargs) -> None:
    kwargs.setdefault("grad", full.GradientArgs(offload_checkpoints=True))
    kwargs.setdefault("optimizer", full.OptimizerArgs(host_offload=True))
    full.setup(checkpoint_dir, out_dir, lora=lora, **kwargs)


full.inherit_cli_signature(setup, {'out_dir': Path('out/finetune/offload-lora'), 'lora': LoRAArgs(), 'grad': full.GradientArgs(offload_checkpoints=True),
                                   'optimizer': full.OptimizerArgs(host_offload=True)})
