"""Small helpers for debugging numerics (``keys_values/tools/debug_utils.py:22-175``)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

QUANTILES = [0.01, 0.5, 0.9, 0.99]
MAX_NUM_CATCHES = 50


def for_debug(x: torch.Tensor) -> torch.Tensor:
    """Detached CPU copy."""
    return x.detach().to("cpu").clone()


def torch_quantile(tensor: torch.Tensor, q: float, dim: Optional[int] = None, *, keepdim: bool = False,
                   interpolation: str = "linear") -> torch.Tensor:
    """One scalar quantile by ``kthvalue`` (``torch.quantile`` refuses inputs above 16M entries and
    sorts everything): the two neighbouring order statistics are selected and interpolated."""
    if not 0.0 <= q <= 1.0:
        raise ValueError(f"q = {q} must be in [0, 1]")
    x = tensor.flatten() if dim is None else tensor
    d = 0 if dim is None else dim
    n = x.shape[d]
    pos = q * (n - 1)
    lo, hi = int(pos), min(int(pos) + 1, n - 1)
    if interpolation == "lower":
        ks, w = [lo], 0.0
    elif interpolation == "higher":
        ks, w = [hi if pos > lo else lo], 0.0
    elif interpolation == "nearest":
        ks, w = [round(pos)], 0.0
    elif interpolation == "midpoint":
        ks, w = [lo, hi if pos > lo else lo], 0.5
    elif interpolation == "linear":
        ks, w = [lo, hi], pos - lo
    else:
        raise ValueError(f"interpolation = {interpolation} not supported")
    xf = x.float() if not x.is_floating_point() or x.dtype in (torch.bfloat16, torch.float16) else x
    vals = [xf.kthvalue(k + 1, dim=d, keepdim=True).values for k in ks]
    out = vals[0] if len(vals) == 1 else vals[0].lerp(vals[1], w)
    if keepdim:
        return out
    return out.squeeze() if dim is None else out.squeeze(d)


def size_quantiles_internal(x: torch.Tensor, quantiles: List[float]) -> List[float]:
    a = x.detach().flatten().abs()
    return [float(torch_quantile(a, q)) for q in quantiles]


def size_quantiles(x: torch.Tensor) -> str:
    return "|".join(f"{q:.2f}:{v:.2e}" for q, v in zip(QUANTILES, size_quantiles_internal(x, QUANTILES)))


def debug_compare_dicts(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor], sort_key: Optional[Callable[[str], Any]] = None,
                        verbose: bool = False, print_size: bool = False) -> None:
    """``assert_close`` entry by entry; reports up to ``MAX_NUM_CATCHES`` mismatches before raising."""
    if a.keys() != b.keys():
        raise ValueError(f"Names only in A: {sorted(a.keys() - b.keys())}; only in B: {sorted(b.keys() - a.keys())}")
    caught, last = [], None
    width = max((len(k) for k in a), default=0) + 1
    for name in sorted(a, key=sort_key):
        if print_size:
            print(f"    {name + ':':{width + 1}} {size_quantiles(a[name])}")
        elif verbose:
            print("    " + name)
        try:
            torch.testing.assert_close(a[name], b[name])
        except AssertionError as ex:
            last = ex
            caught.append((name, str(ex)))
            if len(caught) >= MAX_NUM_CATCHES:
                break
    if caught:
        print(f"\nCaught {len(caught)} exceptions:")
        for name, msg in caught:
            print(f"\n    [{name}]\n{msg}")
        raise last


def debug_token_positions(index: Optional[torch.Tensor], name: str) -> None:
    """Prints the strides of an index that is not a plain 1-D range broadcast over batch and heads."""
    if index is not None and index.ndim > 1 and any(st != 0 for st in index.stride()[:-1]):
        print(f"{name}: token_positions: {index.stride()}")
