"""Worker for the multi-GPU tests: launched once per rank by ``test_multi_gpu.py``.

Usage: python dist_worker.py <case> <rank> <world> <port> [backend]
Every case compares the framework's own collective / data-parallel path with the
single-process result or with NCCL, and prints ``OK`` on success.
"""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main():
    case, rank, world, port = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    if cuda:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        globals()["case_" + case](rank, world, dev)
        dist.barrier()
        if rank == 0:
            print("OK", flush=True)
    finally:
        dist.destroy_process_group()


def case_allreduce(rank, world, dev):
    """Fused peer-memory all-reduce (mean) against NCCL, several sizes and offsets."""
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.parallel.symm import SymmetricArena

    for dtype in (torch.bfloat16, torch.float32):
        n = 1_000_003
        arena = SymmetricArena(n, dtype, dev, world, rank)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        for start, end in ((0, n), (1024, 500_000), (8, 24), (999_000, n)):
            x = torch.randn(n, device=dev, dtype=torch.float32, generator=g)
            arena.tensor.copy_(x.to(dtype))
            ref = arena.tensor.float().clone()
            dist.all_reduce(ref, op=dist.ReduceOp.SUM)
            ref /= world
            arena.all_reduce_mean_(start, end)
            torch.cuda.synchronize(dev)
            cu.check_status(dev)
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
            torch.testing.assert_close(arena.tensor[start:end].float(), ref[start:end], atol=tol, rtol=tol)
        # identical bits on every rank
        mine = arena.tensor.clone()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        a = 1024 // (16 // mine.element_size()) * (16 // mine.element_size())
        for other in gathered:
            assert torch.equal(other[a:500_000], mine[a:500_000])
        arena.close()


def case_dp_train(rank, world, dev):
    """Data-parallel LoRA step: gradients after the reducer equal the mean of the per-rank
    gradients computed without it."""
    from keys_values_b200.finetune.engine import build_lora_training_setup

    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    kw = dict(cache_name="h2o-torch-quantized8", cache_length=128, chunk_size=32, lora_r=4, lora_alpha=8, micro_batch_size=1,
              yarn_rope=False, seed=7)
    name = "tiny-qwen3" if dev.type == "cuda" else "tiny-gpt"
    setup = build_lora_training_setup(name, dev, dtype, world_size=world, rank=rank, **kw)
    solo = build_lora_training_setup(name, dev, dtype, world_size=1, rank=0, **kw)
    solo.gpt_model.load_state_dict(setup.gpt_model.state_dict())
    gen = torch.Generator().manual_seed(50 + rank)
    ids = torch.randint(0, setup.config.vocab_size, (1, 384), generator=gen).to(dev)
    tg = torch.randint(0, setup.config.vocab_size, (1, 64), generator=gen).to(dev)
    # reference: local gradients, averaged with the library collective
    solo.optimizer.zero_grad()
    solo.model(ids, tg).backward()
    ref = {}
    for n, p in solo.gpt_model.named_parameters():
        if p.grad is not None:
            g = p.grad.float().clone()
            dist.all_reduce(g, op=dist.ReduceOp.SUM)
            ref[n] = g / world
    setup.grad_reducer.begin_step()
    setup.grad_reducer.flat.zero_()
    setup.model(ids, tg).backward()
    setup.grad_reducer.finish_step()
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
        from keys_values_b200.ops import cuda as cu

        cu.check_status(dev)
    assert ref, "no gradients"
    for n, p in setup.gpt_model.named_parameters():
        if n in ref:
            tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
            torch.testing.assert_close(p.grad.float(), ref[n], atol=tol, rtol=tol, msg=lambda m: f"{n}: {m}")


if __name__ == "__main__":
    main()
