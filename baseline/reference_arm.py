"""Reference arm of ``bench.py``: the unmodified reference library from ``baseline/_ref``.

The reference imports LitGPT (and Lightning for its CLIs) at module import time; neither
is installed in this image and no wheel is available offline, so the library cannot be
imported. The arm then reports ``unavailable`` and exits 0, as the benchmark contract
asks. Nothing of this repository's models, kernels or engine is used on this path.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

REF_ROOT = Path(__file__).resolve().parent / "_ref"


def _probe() -> str:
    if not (REF_ROOT / "keys_values").is_dir():
        return "baseline/_ref is missing (the offline pip install of the reference with --target baseline/_ref was not run)"
    for mod in ("litgpt", "lightning", "jsonargparse"):
        try:
            importlib.import_module(mod)
        except Exception:
            return (f"the reference needs the '{mod}' package at import time (keys_values/config.py imports litgpt.config); "
                    "it is not installed and no wheel is available offline")
    return ""


def run_reference(args) -> dict:
    why = _probe()
    if why:
        return {"impl": "reference", "unavailable": why}
    sys.path.insert(0, str(REF_ROOT))
    try:
        importlib.import_module("keys_values.kvcache.gradient.main")
    except Exception as ex:  # pragma: no cover
        return {"impl": "reference", "unavailable": f"import of the reference failed: {type(ex).__name__}: {ex}"[:300]}
    return {"impl": "reference", "unavailable": "reference imports, but no driver for it is wired in this build"}
