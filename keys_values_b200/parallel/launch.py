"""Process launcher: one process per GPU of one node.

If the environment already describes a rank (``RANK``/``WORLD_SIZE`` from ``torchrun``), the
function is called in this process after ``init_process_group``; otherwise ``devices``
processes are spawned with ``torch.multiprocessing`` and rendezvous on 127.0.0.1. NCCL on
GPUs, gloo on CPU. Role of Fabric's ``launch`` in ``keys_values/finetune/longcontext_full.py:520-571``."""
from __future__ import annotations

import os
import socket
from typing import Any, Callable

import torch
import torch.distributed as dist


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank: int, world_size: int) -> None:
    if world_size > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world_size)


def _worker(local_rank: int, fn: Callable, world_size: int, port: int, kwargs: dict) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(local_rank), LOCAL_RANK=str(local_rank),
                      WORLD_SIZE=str(world_size))
    _init(local_rank, world_size)
    try:
        fn(local_rank, local_rank, world_size, **kwargs)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def launch(fn: Callable[..., Any], devices: int, **kwargs: Any) -> None:
    """Run ``fn(rank, local_rank, world_size, **kwargs)`` on ``devices`` ranks."""
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        _init(rank, world)
        try:
            fn(rank, int(os.environ.get("LOCAL_RANK", rank)), world, **kwargs)
        finally:
            if dist.is_initialized():
                dist.destroy_process_group()
        return
    if devices == 1:
        fn(0, 0, 1, **kwargs)
        return
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(fn, devices, _free_port(), kwargs), nprocs=devices, join=True)
