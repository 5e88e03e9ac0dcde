"""Rank, device and scalar collectives for code that may run with or without a process group
(``keys_values/optimize/grad_accumulate.py:24-82``). The gradient all-reduce itself is
:class:`keys_values_b200.parallel.dp.GradientReducer` (the reference's
``CPUOffloadAccumulateGradients``): one fused kernel over peer memory instead of flatten → NCCL →
scatter back.
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from keys_values_b200.parallel.dp import GradientReducer as CPUOffloadAccumulateGradients  # noqa: F401


class DistributedPrimitives:
    """Static helpers; everything degrades to a single process when no group is initialised."""

    @staticmethod
    def _active() -> bool:
        return dist.is_available() and dist.is_initialized()

    @staticmethod
    def world_size() -> int:
        return dist.get_world_size() if DistributedPrimitives._active() else 1

    @staticmethod
    def rank() -> int:
        return dist.get_rank() if DistributedPrimitives._active() else 0

    @staticmethod
    def device() -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def _check(x: torch.Tensor) -> None:
        if torch.cuda.is_available() and dist.get_backend() == "nccl" and x.device != DistributedPrimitives.device():
            raise ValueError(f"x.device = {x.device}, must be {DistributedPrimitives.device()}")

    @staticmethod
    def all_reduce_sum(x: torch.Tensor, group=None) -> None:
        if DistributedPrimitives._active() and DistributedPrimitives.world_size() > 1:
            DistributedPrimitives._check(x)
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)

    @staticmethod
    def all_reduce_mean(x: torch.Tensor, group=None) -> None:
        if DistributedPrimitives._active() and DistributedPrimitives.world_size() > 1:
            DistributedPrimitives._check(x)
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)  # gloo has no AVG
            x /= dist.get_world_size(group)

    @staticmethod
    def barrier(group=None) -> None:
        if DistributedPrimitives._active():
            dist.barrier(group=group)
