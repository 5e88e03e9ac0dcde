"""Command line: ``python -m keys_values_b200 <command> [--flag value | --group.field value] …``

Commands (``keys_values/__main__.py:38-47``): ``finetune_long_full``, ``finetune_long_lora``,
``finetune_offload_full``, ``finetune_offload_lora``, ``eval_long``, ``eval_long_ext``,
``recomp_val_losses``, plus ``generate``. Every command maps to a ``setup(...)`` function;
dataclass parameters are filled from dotted flags, ``--config file.yaml`` supplies defaults.
Output is teed to ``$KEYSVALS_LOG_DIR/gpu{LOCAL_RANK}.log`` when that variable is set."""
from __future__ import annotations

import dataclasses
import inspect
import os
import sys
import typing
from pathlib import Path
from typing import Any, Callable, Dict, List

import yaml


def _commands() -> Dict[str, Callable]:
    from keys_values_b200.evaluation import longcontext_eval, longcontext_eval_ext
    from keys_values_b200.finetune import longcon_offload_full, longcon_offload_lora, longcontext_full, longcontext_lora
    from keys_values_b200.generate import base as generate_base
    from keys_values_b200.tools import convert_hf_checkpoint, recompute_val_losses

    return {
        "finetune_long_full": longcontext_full.setup,
        "finetune_long_lora": longcontext_lora.setup,
        "finetune_offload_full": longcon_offload_full.setup,
        "finetune_offload_lora": longcon_offload_lora.setup,
        "eval_long": longcontext_eval.setup,
        "eval_long_ext": longcontext_eval_ext.setup,
        "recomp_val_losses": recompute_val_losses.setup,
        "generate": generate_base.main,
        "convert_hf_checkpoint": convert_hf_checkpoint.setup,
    }


PARSER_DATA = ("finetune_long_full", "finetune_long_lora", "finetune_offload_full", "finetune_offload_lora", "eval_long", "eval_long_ext",
               "recomp_val_losses", "generate", "convert_hf_checkpoint")


class TeeOutput:
    def __init__(self, stream, path: Path):
        self.stream, self.fp = stream, open(path, "a", buffering=1)

    def write(self, data):
        self.stream.write(data)
        self.fp.write(data)

    def flush(self):
        self.stream.flush()
        self.fp.flush()

    def isatty(self):
        return False


def _setup_rank_logs() -> None:
    log_dir = os.environ.get("KEYSVALS_LOG_DIR") or os.environ.get("VALKEYRIE_LOG_DIR")
    if not log_dir:
        return
    Path(log_dir).mkdir(parents=True, exist_ok=True)
    path = Path(log_dir) / f"gpu{os.environ.get('LOCAL_RANK', '0')}.log"
    sys.stdout = TeeOutput(sys.stdout, path)
    sys.stderr = TeeOutput(sys.stderr, path)


def _convert(value: str, annotation: Any) -> Any:
    origin = typing.get_origin(annotation)
    args = [a for a in typing.get_args(annotation) if a is not type(None)]
    if value in ("null", "None", "none") and (origin is typing.Union or annotation is Any):
        return None
    if origin is typing.Union and args:
        for a in args:
            try:
                return _convert(value, a)
            except (ValueError, TypeError):
                continue
        return value
    if annotation is bool:
        if value.lower() in ("true", "1", "yes"):
            return True
        if value.lower() in ("false", "0", "no"):
            return False
        raise ValueError(value)
    if annotation in (int, float, str):
        return annotation(value)
    if annotation is Path:
        return Path(value)
    return yaml.safe_load(value)


def _resolved_hints(fn) -> Dict[str, Any]:
    try:
        return typing.get_type_hints(fn)
    except Exception:
        return {n: p.annotation for n, p in inspect.signature(fn).parameters.items()}


def build_kwargs(fn: Callable, argv: List[str]) -> Dict[str, Any]:
    """Map ``--name value`` / ``--group.field value`` / positionals onto ``fn``'s parameters."""
    sig = inspect.signature(fn)
    hints = _resolved_hints(fn)
    values: Dict[str, Any] = {}
    nested: Dict[str, Dict[str, str]] = {}
    positionals = [n for n, p in sig.parameters.items() if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    i, pos_i = 0, 0
    file_cfg: Dict[str, Any] = {}
    while i < len(argv):
        tok = argv[i]
        if tok == "--config":
            file_cfg = yaml.safe_load(Path(argv[i + 1]).read_text()) or {}
            i += 2
        elif tok.startswith("--"):
            key = tok[2:]
            if "=" in key:
                key, val = key.split("=", 1)
                i += 1
            else:
                val = argv[i + 1]
                i += 2
            if "." in key:
                g, f = key.split(".", 1)
                nested.setdefault(g, {})[f] = val
            else:
                values[key] = val
        else:
            values[positionals[pos_i]] = tok
            pos_i += 1
            i += 1
    for k, v in file_cfg.items():
        if isinstance(v, dict) and k in sig.parameters and dataclasses.is_dataclass(_dc_type(hints.get(k))):
            for f, fv in v.items():
                nested.setdefault(k, {}).setdefault(f, fv)
        else:
            values.setdefault(k, v)
    out: Dict[str, Any] = {}
    for name, raw in values.items():
        ann = hints.get(name, Any)
        out[name] = _convert(raw, ann) if isinstance(raw, str) else raw
    for g, fields_ in nested.items():
        dc = _dc_type(hints.get(g))
        if dc is None:
            raise SystemExit(f"unknown argument group --{g}.*")
        fh = _resolved_hints(dc)
        out[g] = dc(**{f: (_convert(v, fh.get(f, Any)) if isinstance(v, str) else v) for f, v in fields_.items()})
    return out


def _dc_type(annotation: Any):
    if annotation is None:
        return None
    if dataclasses.is_dataclass(annotation):
        return annotation
    for a in typing.get_args(annotation):
        if dataclasses.is_dataclass(a):
            return a
    return None


def main(argv=None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: python -m keys_values_b200 <command> [args]\ncommands: " + ", ".join(PARSER_DATA))
        return
    cmds = _commands()
    if argv[0] not in cmds:
        raise SystemExit(f"unknown command {argv[0]!r}; choose from {', '.join(cmds)}")
    _setup_rank_logs()
    import torch

    torch.set_float32_matmul_precision("high")
    fn = cmds[argv[0]]
    fn(**build_kwargs(fn, argv[1:]))


if __name__ == "__main__":
    main()
