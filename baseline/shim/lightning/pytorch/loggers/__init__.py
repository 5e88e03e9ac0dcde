import csv
import os
from typing import Any, Dict, Optional


class CSVLogger:
    def __init__(self, root_dir: Any = ".", name: str = "logs", flush_logs_every_n_steps: int = 1, **kwargs: Any) -> None:
        self.log_dir = os.path.join(str(root_dir), name)
        self.rows = []

    def log_metrics(self, metrics: Dict[str, Any], step: Optional[int] = None) -> None:
        self.rows.append(dict(metrics, step=step))
        os.makedirs(self.log_dir, exist_ok=True)
        keys = sorted({k for r in self.rows for k in r})
        with open(os.path.join(self.log_dir, "metrics.csv"), "w", newline="") as fp:
            writer = csv.DictWriter(fp, fieldnames=keys)
            writer.writeheader()
            writer.writerows(self.rows)

    def log_hyperparams(self, params: Any) -> None:
        pass
