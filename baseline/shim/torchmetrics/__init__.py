"""Stand-in for ``torchmetrics``: ``RunningMean`` over a window of the last values."""
from collections import deque

import torch


class RunningMean:
    def __init__(self, window: int = 5, sync_on_compute: bool = False, **kwargs) -> None:
        self.values = deque(maxlen=window)
        self.device = torch.device("cpu")

    def to(self, device):
        self.device = torch.device(device)
        return self

    def update(self, value) -> None:
        self.values.append(torch.as_tensor(value, dtype=torch.float32).detach().to(self.device))

    def compute(self) -> torch.Tensor:
        if not self.values:
            return torch.tensor(float("nan"), device=self.device)
        return torch.stack(list(self.values)).mean()

    def reset(self) -> None:
        self.values.clear()
