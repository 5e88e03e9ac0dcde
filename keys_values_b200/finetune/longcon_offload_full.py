"""``finetune_offload_full``: as ``finetune_long_full``, with what only the optimizer touches (fp32 master
weights, fp32 gradients, optimizer moments: 16 bytes per parameter for AdamW) in pinned host memory
(:class:`keys_values_b200.optimize.host_optimizer.HostOffloadOptimizer`) and the activation / KV
checkpoints of the step on the host as well. The bf16 weights and gradients stay on the device.

The reference keeps the weights themselves on the host and copies shards to the GPU for every row of
the backward pass (``keys_values/finetune/longcon_offload_full.py``, ``gradient/main.py:1100-1301``);
shard copies of a host model are available here too (:mod:`keys_values_b200.optimize.model_factory`)."""
from __future__ import annotations

from pathlib import Path
from typing import Union

from keys_values_b200.finetune import longcontext_full as full


def setup(checkpoint_dir: Union[str, Path], out_dir: Union[str, Path] = Path("out/finetune/offload-full"), **kwargs) -> None:
    kwargs.setdefault("grad", full.GradientArgs(offload_checkpoints=True))
    kwargs.setdefault("optimizer", full.OptimizerArgs(host_offload=True))
    full.setup(checkpoint_dir, out_dir, **kwargs)


full.inherit_cli_signature(setup, {'out_dir': Path('out/finetune/offload-full'), 'grad': full.GradientArgs(offload_checkpoints=True),
                                   'optimizer': full.OptimizerArgs(host_offload=True)})
