"""Worker of the host-side failure-detection tests (gloo ranks on CPU, no GPU involved).

Usage: python health_worker.py <case> <rank> <world> <port>
  exit  : rank 1 leaves silently between steps 1 and 2; the others must detect the missing heartbeat
  raise : rank 1 hits an exception in step 2, reports it and leaves; the others must see the report
Prints ``DETECTED <ranks>`` on the surviving ranks.
"""
import os
import sys
from datetime import timedelta
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist

from keys_values_b200.parallel.health import RankFailure, RankHealth


def main():
    case, rank, world, port = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    health = RankHealth(rank, world)
    x = torch.ones(4)
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                if case == "raise":
                    try:
                        raise ValueError("injected host failure")
                    except ValueError as ex:
                        health.mark_failed(repr(ex))
                os._exit(0)  # leaves between steps: nothing of this rank is in flight
            health.enter_step(step, grace_s=8.0)  # host rendezvous before this step's collectives
            dist.all_reduce(x)
        print("NOT DETECTED", flush=True)
    except RankFailure as ex:
        print("DETECTED", sorted(ex.ranks), next(iter(ex.ranks.values())), flush=True)
    if rank == 0:
        import time

        time.sleep(3.0)  # this process serves the key-value store: the other survivors are still reading it
    os._exit(0)  # the group cannot be torn down collectively any more


if __name__ == "__main__":
    main()
