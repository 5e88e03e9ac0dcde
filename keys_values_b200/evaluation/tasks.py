"""Evaluation job grid claimed through lock files (``keys_values/evaluation/tasks.py:44-278``).

A *task* is (setup, checkpoint); its batches are numbered. Any number of worker processes may
run the same command: a worker claims a batch by creating ``.../batch_<n>.lock`` atomically,
writes ``eval_metrics_<n>.csv`` when done, and skips batches whose result or lock exists.
There is no communication between workers, so evaluation restarts for free."""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, List, Optional


@dataclass(frozen=True)
class EvaluationTask:
    setup_name: str
    checkpoint: str

    @property
    def key(self) -> str:
        return f"{self.setup_name}__{Path(self.checkpoint).name}"


class EvaluationTasks:
    def __init__(self, setups: List[str], checkpoints: List[str]):
        self.tasks = [EvaluationTask(s, c) for s in setups for c in checkpoints]

    def __iter__(self) -> Iterator[EvaluationTask]:
        return iter(self.tasks)

    def __len__(self) -> int:
        return len(self.tasks)


class EvaluationWithTasksHelper:
    def __init__(self, out_dir: Path, eval_dir: str = "eval"):
        self.out_dir, self.eval_dir = Path(out_dir), eval_dir

    def task_dir(self, task: EvaluationTask) -> Path:
        d = self.out_dir / task.key / self.eval_dir
        d.mkdir(parents=True, exist_ok=True)
        return d

    def result_path(self, task: EvaluationTask, batch_idx: int) -> Path:
        return self.task_dir(task) / f"eval_metrics_{batch_idx}.csv"

    def get_lock(self, task: EvaluationTask, batch_idx: int) -> Optional[Path]:
        """Claim a batch; returns the lock path, or ``None`` if it is done or taken."""
        if self.result_path(task, batch_idx).is_file():
            return None
        lock = self.task_dir(task) / f"batch_{batch_idx}.lock"
        try:
            fd = os.open(str(lock), os.O_CREAT | os.O_EXCL | os.O_WRONLY)
            os.write(fd, str(os.getpid()).encode())
            os.close(fd)
            return lock
        except FileExistsError:
            return None

    def release(self, lock: Path, done: bool) -> None:
        """Remove the lock; if the batch did not finish it becomes claimable again."""
        Path(lock).unlink(missing_ok=True)

    def pending(self, task: EvaluationTask, num_batches: int) -> List[int]:
        return [b for b in range(num_batches) if not self.result_path(task, b).is_file()]
