"""Minimal ``Fabric``: one process per device (started by ``torchrun``), collectives through ``torch.distributed``."""
from __future__ import annotations

import contextlib
import os
import random
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist


def seed_everything(seed: int, workers: bool = False, verbose: bool = False) -> int:
    import numpy as np

    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    return seed


class Fabric:
    def __init__(self, devices: Any = 1, num_nodes: int = 1, strategy: Any = "auto", precision: Optional[str] = None,
                 loggers: Any = None, plugins: Any = None, accelerator: Any = "auto", **kwargs: Any) -> None:
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.global_rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.node_rank = 0
        self.precision = precision
        self.loggers = loggers if isinstance(loggers, (list, tuple)) else ([] if loggers is None else [loggers])
        self.device = torch.device("cuda", self.local_rank) if torch.cuda.is_available() else torch.device("cpu")
        self.strategy = strategy

    @property
    def logger(self):
        return self.loggers[0] if self.loggers else None

    @property
    def is_global_zero(self) -> bool:
        return self.global_rank == 0

    def launch(self, function=None, *args: Any, **kwargs: Any) -> Any:
        if self.world_size > 1 and not dist.is_initialized():
            backend = "nccl" if self.device.type == "cuda" else "gloo"
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
                dist.init_process_group(backend, device_id=self.device)
            else:
                dist.init_process_group(backend)
        if function is not None:
            return function(self, *args, **kwargs)

    def _dtype(self) -> Optional[torch.dtype]:
        return {"bf16-true": torch.bfloat16, "16-true": torch.float16, "32-true": torch.float32}.get(self.precision or "")

    @contextlib.contextmanager
    def init_module(self, empty_init: Optional[bool] = None):
        dtype = self._dtype()
        previous = torch.get_default_dtype()
        if dtype is not None:
            torch.set_default_dtype(dtype)
        try:
            with torch.device(self.device):
                yield
        finally:
            torch.set_default_dtype(previous)

    def init_tensor(self):
        return self.init_module()

    def setup(self, module, *optimizers, **kwargs):
        module = module.to(self.device)
        return (module, *optimizers) if optimizers else module

    def setup_module(self, module, **kwargs):
        return module.to(self.device)

    def setup_optimizers(self, *optimizers):
        return optimizers[0] if len(optimizers) == 1 else optimizers

    def setup_dataloaders(self, *loaders, **kwargs):
        return loaders[0] if len(loaders) == 1 else loaders

    def to_device(self, obj):
        if isinstance(obj, torch.Tensor) or isinstance(obj, torch.nn.Module):
            return obj.to(self.device)
        if isinstance(obj, dict):
            return {k: self.to_device(v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(self.to_device(v) for v in obj)
        return obj

    def all_reduce(self, x: torch.Tensor, reduce_op: str = "mean", group: Any = None) -> torch.Tensor:
        if self.world_size > 1:
            ops = {"mean": dist.ReduceOp.AVG, "avg": dist.ReduceOp.AVG, "sum": dist.ReduceOp.SUM,
                   "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
            op = ops[reduce_op.lower()]
            if op == dist.ReduceOp.AVG and (x.device.type != "cuda" or not x.is_floating_point()):
                dist.all_reduce(x, op=dist.ReduceOp.SUM)
                x.div_(self.world_size) if x.is_floating_point() else x.floor_divide_(self.world_size)
            else:
                dist.all_reduce(x, op=op)
        return x

    def broadcast(self, obj: Any, src: int = 0) -> Any:
        if self.world_size > 1:
            box = [obj]
            dist.broadcast_object_list(box, src=src)
            return box[0]
        return obj

    def barrier(self, name: Optional[str] = None) -> None:
        if self.world_size > 1:
            dist.barrier()

    @contextlib.contextmanager
    def rank_zero_first(self, local: bool = False):
        if self.global_rank != 0:
            self.barrier()
        yield
        if self.global_rank == 0:
            self.barrier()

    def print(self, *args: Any, **kwargs: Any) -> None:
        if self.global_rank == 0:
            print(*args, **kwargs)

    def seed_everything(self, seed: int, workers: bool = False) -> int:
        return seed_everything(seed)

    def backward(self, tensor: torch.Tensor, *args: Any, **kwargs: Any) -> None:
        tensor.backward(*args, **kwargs)

    def clip_gradients(self, module, optimizer, max_norm=None, clip_val=None, **kwargs):
        if max_norm is not None:
            return torch.nn.utils.clip_grad_norm_(module.parameters(), max_norm)

    def save(self, path, state: Dict[str, Any], filter: Optional[Dict[str, Any]] = None) -> None:
        if self.global_rank != 0:
            return
        out = {}
        for key, value in state.items():
            value = value.state_dict() if hasattr(value, "state_dict") else value
            if filter is not None and key in filter and isinstance(value, dict):
                value = {k: v for k, v in value.items() if filter[key](k, v)}
            out[key] = value
        os.makedirs(os.path.dirname(str(path)) or ".", exist_ok=True)
        torch.save(out, str(path))

    def load(self, path, state: Optional[Dict[str, Any]] = None, strict: bool = True) -> Dict[str, Any]:
        loaded = torch.load(str(path), map_location="cpu", weights_only=False)
        if state is None:
            return loaded
        for key, value in list(state.items()):
            if key in loaded and hasattr(value, "load_state_dict"):
                value.load_state_dict(loaded.pop(key))
            elif key in loaded:
                state[key] = loaded.pop(key)
        return loaded

    def load_raw(self, path, obj, strict: bool = True) -> None:
        obj.load_state_dict(torch.load(str(path), map_location="cpu", weights_only=False), strict=strict)

    def log_dict(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        for logger in self.loggers:
            if hasattr(logger, "log_metrics"):
                logger.log_metrics(metrics, step=step)

    def log(self, name: str, value: Any, step: Optional[int] = None) -> None:
        self.log_dict({name: value}, step=step)
