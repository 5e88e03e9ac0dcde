"""Index helpers, NaN checks, precision names, memory messages, file-locked CSV append."""
from __future__ import annotations

import csv
import enum
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch

__all__ = [
    "VerbosityLevels", "index_to_3d", "expand_index", "is_index_1d", "repeat_interleave", "copy_parameters", "check_for_nan",
    "check_for_nan_module_weights", "str_to_torch_dtype", "get_default_supported_precision", "message_memory_all_devices",
    "nested_get", "nested_set", "flush_io_streams", "append_results_to_csv", "num_parameters", "find_multiple", "randint_torch",
]


class VerbosityLevels(str, enum.Enum):
    NONE = "none"
    SOME = "some"
    MORE = "more"
    ALL = "all"


def find_multiple(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


def randint_torch(low: int, high: int) -> int:
    """Random integer in ``[low, high]`` from torch's generator (reproducible with ``manual_seed``)."""
    return int(torch.randint(low, high + 1, (1,)).item())


def index_to_3d(index: torch.Tensor, batch_size: int, n_query_groups: int) -> torch.Tensor:
    """Broadcast a 1-D index to ``(batch_size, n_query_groups, n)`` without copying."""
    assert index.ndim == 1
    return index.view(1, 1, -1).expand(batch_size, n_query_groups, -1)


def expand_index(index: torch.Tensor, head_size: int) -> torch.Tensor:
    return index.unsqueeze(-1).expand(*index.shape, head_size)


def is_index_1d(index: torch.Tensor) -> bool:
    """True if a 3-D index is a stride-0 expansion of a 1-D one."""
    return index.ndim == 3 and index.stride(0) == 0 and index.stride(1) == 0


def repeat_interleave(x: torch.Tensor, n: int) -> torch.Tensor:
    """``(B, G, ...)`` → ``(B, G·n, ...)`` where every group is repeated ``n`` times."""
    if n == 1:
        return x
    B, G = x.shape[:2]
    return x.unsqueeze(2).expand(B, G, n, *x.shape[2:]).reshape(B, G * n, *x.shape[2:])


def copy_parameters(src: torch.nn.Module, dst: torch.nn.Module, non_blocking: bool = True) -> None:
    dst_params = dict(dst.named_parameters())
    for name, p in src.named_parameters():
        dst_params[name].data.copy_(p.data, non_blocking=non_blocking)


def check_for_nan(x: Optional[torch.Tensor], where: str, name: str, extra_msg: Optional[str] = None, do_boom: bool = True) -> bool:
    if x is None:
        return False
    bad = not torch.isfinite(x).all().item()
    if bad:
        msg = f"{where}: {name} has NaN or Inf entries" + (f" ({extra_msg})" if extra_msg else "")
        if do_boom:
            raise AssertionError(msg)
        print(msg)
    return bad


def check_for_nan_module_weights(module: torch.nn.Module, extra_msg: Optional[str] = None, do_grads: bool = False) -> None:
    for name, p in module.named_parameters():
        check_for_nan(p.data, "module", name, extra_msg)
        if do_grads and p.grad is not None:
            check_for_nan(p.grad, "module", name + ".grad", extra_msg)


_PRECISIONS = {
    "32-true": torch.float32, "32": torch.float32, "16-true": torch.float16, "16-mixed": torch.float16,
    "bf16-true": torch.bfloat16, "bf16-mixed": torch.bfloat16, "64-true": torch.float64,
}


def str_to_torch_dtype(precision: str) -> torch.dtype:
    if precision not in _PRECISIONS:
        raise ValueError(f"precision = {precision} not supported; must be in {sorted(_PRECISIONS)}")
    return _PRECISIONS[precision]


def get_default_supported_precision(training: bool) -> str:
    if torch.cuda.is_available() and torch.cuda.is_bf16_supported():
        return "bf16-true"
    return "32-true"


def message_memory_all_devices(prefix: str = "") -> str:
    if not torch.cuda.is_available():
        return prefix + "no CUDA device"
    parts = []
    for d in range(torch.cuda.device_count()):
        alloc = torch.cuda.memory_allocated(d) / 2**30
        peak = torch.cuda.max_memory_allocated(d) / 2**30
        parts.append(f"cuda:{d} allocated {alloc:.2f} GB (peak {peak:.2f} GB)")
    return prefix + "; ".join(parts)


def nested_get(d: Dict[str, Any], dotted: str, default: Any = None) -> Any:
    cur: Any = d
    for k in dotted.split("."):
        if not isinstance(cur, dict) or k not in cur:
            return default
        cur = cur[k]
    return cur


def nested_set(d: Dict[str, Any], dotted: str, value: Any) -> None:
    keys = dotted.split(".")
    cur = d
    for k in keys[:-1]:
        cur = cur.setdefault(k, {})
    cur[keys[-1]] = value


def flush_io_streams() -> None:
    import sys

    sys.stdout.flush()
    sys.stderr.flush()


def append_results_to_csv(results: List[Dict[str, Any]], path: Union[str, Path], timeout: float = 60.0) -> None:
    """Append rows to a CSV shared by several processes (guarded by a lock file)."""
    from filelock import FileLock

    path = Path(path)
    if not results:
        return
    with FileLock(str(path) + ".lock", timeout=timeout):
        exists = path.exists()
        with path.open("a", newline="") as fp:
            writer = csv.DictWriter(fp, fieldnames=list(results[0].keys()))
            if not exists:
                writer.writeheader()
            writer.writerows(results)


def num_parameters(module: torch.nn.Module, requires_grad: Optional[bool] = None) -> int:
    return sum(p.numel() for p in module.parameters() if requires_grad is None or p.requires_grad == requires_grad)
