"""Stand-in for ``litgpt.utils``. Names the benchmark path does not reach resolve to stubs that raise."""
from __future__ import annotations

import inspect
import math
from pathlib import Path
from typing import Any, Dict, Iterable, Optional, Union

import torch
import torch.nn as nn

_BITANDBYTES_AVAILABLE_NOT_EQUAL_0_42_0 = False


def map_old_state_dict_weights(state_dict: Dict, mapping: Dict, prefix: str) -> Dict:
    """Renames ``prefix + old`` keys to ``prefix + new`` in place (checkpoints saved without LoRA wrappers)."""
    for old, new in mapping.items():
        full_old, full_new = prefix + old, prefix + new
        if full_old in state_dict:
            state_dict[full_new] = state_dict.pop(full_old)
    return state_dict


def num_parameters(module: nn.Module, requires_grad: Optional[bool] = None) -> int:
    return sum(p.numel() for p in module.parameters() if requires_grad is None or p.requires_grad == requires_grad)


def get_default_supported_precision(training: bool) -> str:
    if torch.cuda.is_available() and torch.cuda.is_bf16_supported():
        return "bf16-mixed" if training else "bf16-true"
    return "32-true"


def parse_devices(devices: Union[str, int]) -> int:
    if devices in (-1, "auto"):
        return torch.cuda.device_count() or 1
    if isinstance(devices, int) and devices > 0:
        return devices
    raise ValueError(f"Devices must be 'auto' or a positive integer, got: {devices!r}")


def instantiate_torch_optimizer(optimizer, model_parameters, **kwargs):
    if isinstance(optimizer, str):
        cls = getattr(torch.optim, optimizer)
        valid = set(inspect.signature(cls).parameters)
        return cls(model_parameters, **{k: v for k, v in kwargs.items() if k in valid})
    optimizer = dict(optimizer)
    args = dict(optimizer.get("init_args", {}))
    args.update(kwargs)
    module, _, name = optimizer["class_path"].rpartition(".")
    cls = getattr(__import__(module, fromlist=[name]), name)
    valid = set(inspect.signature(cls).parameters)
    return cls(model_parameters, **{k: v for k, v in args.items() if k in valid})


def load_checkpoint(fabric, model: nn.Module, checkpoint_path: Path, strict: bool = True) -> None:
    state = torch.load(str(checkpoint_path), map_location="cpu", weights_only=False)
    model.load_state_dict(state.get("model", state), strict=strict)


def check_valid_checkpoint_dir(checkpoint_dir: Path, *args, **kwargs) -> None:
    if not Path(checkpoint_dir).is_dir():
        raise FileNotFoundError(f"checkpoint_dir {str(checkpoint_dir)!r} is not a directory")


def extend_checkpoint_dir(checkpoint_dir: Path) -> Path:
    return Path(checkpoint_dir)


def auto_download_checkpoint(model_name, *args, **kwargs) -> Path:
    return Path(model_name)


def init_out_dir(out_dir: Path) -> Path:
    return Path(out_dir)


def check_nvlink_connectivity(fabric=None) -> None:
    return None


def check_file_size_on_cpu_and_warn(checkpoint_path, device, size_limit: int = 4_600_000_000) -> int:
    return Path(checkpoint_path).stat().st_size


class CycleIterator:
    """Iterates over an iterable forever, counting completed passes in ``epoch``."""

    def __init__(self, iterable: Iterable) -> None:
        self.iterable = iterable
        self.epoch = 0
        self._iterator = None

    def __next__(self) -> Any:
        if self._iterator is None:
            self._iterator = iter(self.iterable)
        try:
            return next(self._iterator)
        except StopIteration:
            self._iterator = iter(self.iterable)
            self.epoch += 1
            return next(self._iterator)

    def __iter__(self):
        return self


def _stub(name: str):
    def raiser(*args, **kwargs):
        raise NotImplementedError(f"litgpt.utils.{name} is not provided by the stand-in package")

    raiser.__name__ = name
    return raiser


def __getattr__(name: str):
    if name.startswith("__"):
        raise AttributeError(name)
    return _stub(name)
