"""Check gradients recorded on several ranks before and after the gradient all-reduce.

    python -m keys_values_b200.tools.analyze_gradient_data <dir> --iters 0 1 2 --devices 4 [--layers 0 1]

Recording (in a debugging run, with the overlap of the reduction switched off so that the local
gradients still exist when they are recorded):

    from keys_values_b200.tools.analyze_gradient_data import record_gradients, save_record
    before = record_gradients(model, lambda name: "lora_B" in name)      # after backward, before the all-reduce
    ...all-reduce...
    save_record(path, iteration, rank, before, record_gradients(model, lambda name: "lora_B" in name))

The analysis verifies for every iteration that all ranks hold the same keys, that the gradients after the
reduction are identical on all ranks and equal to the mean of the gradients before it, and prints
magnitude quantiles and a text histogram per layer (the reference plots them:
``keys_values/scripts/analyze_gradient_data.py``).
"""
from __future__ import annotations

import argparse
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

import torch

FNAME_MASK = "gradients_iter{iter}_rank{rank}.pt"
PREFIXES = ("before", "after")


def record_gradients(model: torch.nn.Module, predicate: Optional[Callable[[str], bool]] = None) -> Dict[str, torch.Tensor]:
    """CPU copies of the gradients of the parameters whose name passes ``predicate``."""
    return {n: p.grad.detach().float().cpu().clone() for n, p in model.named_parameters()
            if p.grad is not None and (predicate is None or predicate(n))}


def save_record(path: Path, iteration: int, rank: int, before: Dict[str, torch.Tensor], after: Dict[str, torch.Tensor]) -> Path:
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    rec = {f"before:{k}": v for k, v in before.items()}
    rec.update({f"after:{k}": v for k, v in after.items()})
    f = path / FNAME_MASK.format(iter=iteration, rank=rank)
    torch.save(rec, f)
    return f


def load_records(path: Path, iteration: int, num_devices: int) -> List[Dict[str, Dict[str, torch.Tensor]]]:
    out = []
    for rank in range(num_devices):
        rec = torch.load(Path(path) / FNAME_MASK.format(iter=iteration, rank=rank), map_location="cpu", weights_only=True)
        out.append({p: {k[len(p) + 1:]: v for k, v in rec.items() if k.startswith(p + ":")} for p in PREFIXES})
    return out


def check_consistency(records: Sequence[Dict[str, Dict[str, torch.Tensor]]], prefix: str = "", rtol: float = 1e-3, atol: float = 1e-6) -> None:
    """Raises ``ValueError`` with the first inconsistency found."""
    keys = set(records[0]["before"])
    for r, rec in enumerate(records):
        for part in PREFIXES:
            if set(rec[part]) != keys:
                raise ValueError(f"{prefix}: rank {r} [{part}] has other keys than rank 0 [before]: {sorted(set(rec[part]) ^ keys)[:5]}")
    for name in sorted(keys):
        mean = torch.stack([rec["before"][name] for rec in records]).mean(0)
        for r, rec in enumerate(records):
            if not torch.equal(rec["after"][name], records[0]["after"][name]):
                raise ValueError(f"{prefix}: '{name}' after the reduction differs between rank 0 and rank {r}")
        if not torch.allclose(records[0]["after"][name], mean, rtol=rtol, atol=atol + rtol * float(mean.abs().max())):
            err = float((records[0]["after"][name] - mean).abs().max())
            raise ValueError(f"{prefix}: '{name}' after the reduction is not the mean of the ranks (max abs difference {err:.3e})")


def text_histogram(x: torch.Tensor, bins: int = 12, width: int = 40) -> str:
    """Histogram of ``log10 |x|`` (zeros counted separately), one line per bin."""
    a = x.flatten().abs()
    nz = a[a > 0]
    lines = [f"  zeros: {int((a == 0).sum())} of {a.numel()}"]
    if nz.numel():
        lg = nz.log10()
        lo, hi = float(lg.min()), float(lg.max())
        hist = torch.histc(lg, bins=bins, min=lo, max=hi if hi > lo else lo + 1)
        top = float(hist.max())
        for i, c in enumerate(hist.tolist()):
            edge = lo + (hi - lo) * i / bins
            lines.append(f"  1e{edge:+6.2f} | {'#' * int(round(width * c / top))} {int(c)}")
    return "\n".join(lines)


def main(argv=None) -> None:
    from keys_values_b200.tools.debug_utils import size_quantiles

    ap = argparse.ArgumentParser()
    ap.add_argument("path", type=Path)
    ap.add_argument("--iters", type=int, nargs="+", required=True)
    ap.add_argument("--devices", type=int, required=True)
    ap.add_argument("--layers", type=int, nargs="*", default=[])
    a = ap.parse_args(argv)
    for it in a.iters:
        records = load_records(a.path, it, a.devices)
        check_consistency(records, prefix=f"iteration {it}")
        print(f"iteration {it}: {len(records[0]['before'])} tensors consistent over {a.devices} ranks")
        for layer in a.layers:
            names = [n for n in sorted(records[0]["after"]) if f"transformer.h.{layer}." in n]
            if names:
                x = torch.cat([records[0]["after"][n].flatten() for n in names])
                print(f" layer {layer}: |g| quantiles {size_quantiles(x)}")
                print(text_histogram(x))


if __name__ == "__main__":
    main()
