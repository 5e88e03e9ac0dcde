"""``recomp_val_losses``: recompute validation losses of the checkpoints of a run with another
KV-cache setup (``keys_values/scripts/recompute_val_losses.py``); uses the evaluation job grid."""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Union

from keys_values_b200.evaluation import longcontext_eval_ext as ext
from keys_values_b200.finetune.args import EvalArgs, KVCacheArgs


def setup(out_dir: Union[str, Path], data=None, kv_cache: Optional[KVCacheArgs] = None, devices: int = 1, eval: EvalArgs = EvalArgs(),
          eval_dir: str = "recomputed") -> None:
    out_dir = Path(out_dir)
    ckpts = sorted(p.name for p in out_dir.glob("step-*")) + (["final"] if (out_dir / "final").is_dir() else [])
    ext.setup(out_dir, checkpoints=ckpts, data=data, kv_cache=kv_cache, eval=eval, devices=devices, eval_dir=eval_dir)
