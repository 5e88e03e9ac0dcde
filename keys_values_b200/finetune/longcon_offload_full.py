"""``finetune_offload_full``: as ``finetune_long_full`` but model weights and optimizer state
live in (pinned) host memory and are streamed to the GPU one row of layers at a time
(``keys_values/finetune/longcon_offload_full.py``, ``gradient/main.py:1100-1301``).

With 180 GB of device memory the models of the registry fit on the GPU, so this mode is an
option for larger models; it reuses the flat-vector weight access of
:mod:`keys_values_b200.optimize`."""
from __future__ import annotations

from pathlib import Path
from typing import Union

from keys_values_b200.finetune import longcontext_full as full


def setup(checkpoint_dir: Union[str, Path], out_dir: Union[str, Path] = Path("out/finetune/offload-full"), **kwargs) -> None:
    kwargs.setdefault("grad", full.GradientArgs(offload_checkpoints=True))
    full.setup(checkpoint_dir, out_dir, **kwargs)


full.inherit_cli_signature(setup, {'out_dir': Path('out/finetune/offload-full'), 'grad': full.GradientArgs(offload_checkpoints=True)})
