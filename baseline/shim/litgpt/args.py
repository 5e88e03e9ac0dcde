"""Stand-in for ``litgpt.args``."""
from dataclasses import dataclass
from typing import Optional


@dataclass
class EvalArgs:
    interval: int = 600
    max_new_tokens: Optional[int] = None
    max_iters: int = 100
    initial_validation: bool = False
    final_validation: bool = True
    evaluate_example: str = "first"


@dataclass
class TrainArgs:
    save_interval: Optional[int] = 1000
    log_interval: int = 1
    global_batch_size: int = 64
    micro_batch_size: int = 4
    lr_warmup_steps: Optional[int] = 100
    lr_warmup_fraction: Optional[float] = None
    epochs: Optional[int] = None
    max_tokens: Optional[int] = None
    max_steps: Optional[int] = None
    max_time: Optional[float] = None
    max_seq_length: Optional[int] = None
    tie_embeddings: Optional[bool] = None
    max_norm: Optional[float] = None
    min_lr: float = 6e-5

    def gradient_accumulation_iters(self, devices: int, num_nodes: int = 1) -> int:
        return self.batch_size(devices, num_nodes) // self.micro_batch_size

    def batch_size(self, devices: int, num_nodes: int = 1) -> int:
        return self.global_batch_size // (devices * num_nodes)

    def warmup_iters(self, devices: int, num_nodes: int, max_iters: int, train_dataloader) -> int:
        if self.lr_warmup_fraction:
            return min(max_iters, int(self.lr_warmup_fraction * max_iters) + 1)
        return min(max_iters, (self.lr_warmup_steps or 0) * self.gradient_accumulation_iters(devices, num_nodes))
