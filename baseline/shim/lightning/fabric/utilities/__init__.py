from typing import Any, Dict


class ThroughputMonitor:
    """Accumulates ``update(**counters)`` calls; ``compute_and_log`` returns what was last given."""

    def __init__(self, fabric: Any = None, **kwargs: Any) -> None:
        self.fabric = fabric
        self.last: Dict[str, Any] = {}

    def update(self, **kwargs: Any) -> None:
        self.last = dict(kwargs)

    def compute(self) -> Dict[str, Any]:
        out = {}
        t = self.last.get("time")
        if t:
            for key in ("batches", "samples", "lengths"):
                if key in self.last:
                    out[f"throughput/{key}_per_sec"] = self.last[key] / t
        return out

    def compute_and_log(self, step: Any = None, **kwargs: Any) -> Dict[str, Any]:
        self.update(**kwargs) if kwargs else None
        metrics = self.compute()
        if self.fabric is not None and metrics:
            self.fabric.log_dict(metrics, step=step)
        return metrics
