"""Training-state checkpoints for ``--resume`` (``keys_values/finetune/resume_state.py:61-266``).

Files in a step directory: ``training_state_optimizer.pth`` (optimizer + scheduler state),
``training_state.pth`` (iteration counters and the data-module state),
``training_state_iterator_rank{r}.pth`` (the sampler position of every rank). Only the
last ``training_state_num`` checkpoints keep these files."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, List, Optional

import torch

OPT_FNAME = "training_state_optimizer.pth"
STATE_FNAME = "training_state.pth"
ITER_FNAME = "training_state_iterator_rank{rank}.pth"


class TrainingStateManager:
    def __init__(self, out_dir: Path, rank: int = 0, world_size: int = 1, training_state_num: int = 3, tp_rank: Optional[int] = None):
        """``tp_rank``: under tensor parallelism every shard has its own optimizer state; the ranks of the first
        replica (``rank == tp_rank``) write one optimizer file each."""
        self.out_dir, self.rank, self.world_size, self.training_state_num = Path(out_dir), rank, world_size, training_state_num
        self.tp_rank = tp_rank
        self._saved: List[Path] = []

    def save(self, step_dir: Path, optimizer, scheduler, iter_num: int, step_count: int, data_state: Optional[Dict[str, Any]],
             iterator_state: Optional[Dict[str, Any]], extra: Optional[Dict[str, Any]] = None) -> None:
        step_dir = Path(step_dir)
        step_dir.mkdir(parents=True, exist_ok=True)
        torch.save(iterator_state or {}, step_dir / ITER_FNAME.format(rank=self.rank))
        if self.tp_rank is not None and self.rank == self.tp_rank and self.rank != 0:
            torch.save({"optimizer": optimizer.state_dict(), "scheduler": None}, step_dir / opt_fname(self.tp_rank))
        if self.rank == 0:
            torch.save({"optimizer": optimizer.state_dict(), "scheduler": None if scheduler is None else scheduler.state_dict()}, step_dir / OPT_FNAME)
            torch.save({"iter_num": iter_num, "step_count": step_count, "world_size": self.world_size, "data": data_state or {},
                        **(extra or {})}, step_dir / STATE_FNAME)
            self._saved.append(step_dir)
            while len(self._saved) > self.training_state_num:
                old = self._saved.pop(0)
                for f in [OPT_FNAME, STATE_FNAME] + [ITER_FNAME.format(rank=r) for r in range(self.world_size)]:
                    (old / f).unlink(missing_ok=True)


def opt_fname(tp_rank: Optional[int]) -> str:
    """Optimizer file of a shard: the plain name for shard 0 (and without tensor parallelism)."""
    return OPT_FNAME if not tp_rank else OPT_FNAME.replace(".pth", f"_tp{tp_rank}.pth")


def load_training_state(step_dir: Path) -> Dict[str, Any]:
    return torch.load(str(Path(step_dir) / STATE_FNAME), map_location="cpu", weights_only=False)


def restore_from_training_state(step_dir: Path, optimizer, scheduler, rank: int, world_size: int, tp_rank: Optional[int] = None) -> Dict[str, Any]:
    step_dir = Path(step_dir)
    state = load_training_state(step_dir)
    if state.get("world_size", world_size) != world_size:
        raise ValueError(f"checkpoint was written with {state['world_size']} devices, now running with {world_size}")
    opt = torch.load(str(step_dir / opt_fname(tp_rank)), map_location="cpu", weights_only=False)
    optimizer.load_state_dict(opt["optimizer"])
    sched = opt.get("scheduler")
    if sched is None and tp_rank:
        sched = torch.load(str(step_dir / OPT_FNAME), map_location="cpu", weights_only=False).get("scheduler")
    if scheduler is not None and sched is not None:
        scheduler.load_state_dict(sched)
    it_path = step_dir / ITER_FNAME.format(rank=rank)
    state["iterator"] = torch.load(str(it_path), map_location="cpu", weights_only=False) if it_path.is_file() else {}
    return state


def find_resume_dir(out_dir: Path, resume) -> Optional[Path]:
    """``resume``: ``True``/``"auto"`` → latest ``step-*`` directory that has a training state."""
    if not resume:
        return None
    if isinstance(resume, (str, Path)) and str(resume) not in ("auto", "True", "true"):
        return Path(resume)
    cands = sorted(p for p in Path(out_dir).glob("step-*") if (p / STATE_FNAME).is_file())
    return cands[-1] if cands else None
