"""Long-context LoRA training step with the model sharded over GPUs (tensor parallel), optionally in several
data-parallel replicas.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m keys_values_b200.tools.tp_train_bench --tp 8            # one replica over 8 GPUs
    python -m torch.distributed.run ... --nproc-per-node 8 -m keys_values_b200.tools.tp_train_bench --tp 4   # 2 x 4

Defaults: Qwen3-14B architecture (random-init bf16), 65536-token uniform-random sequences with the loss on the
last 512 tokens, LoRA r=16 on all linears, H2O cache of 8192 slots with int8 storage, chunks of 512, the quantized
cache storage in pinned host memory (``--no-kv-offload`` keeps it on the device). Every replica gets its own
sequence. Device-timed (CUDA events), maximum over ranks; one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen3-14B")
    ap.add_argument("--tp", type=int, default=None, help="ranks per replica (default: all launched ranks)")
    ap.add_argument("--seq-len", type=int, default=65536)
    ap.add_argument("--cache-length", type=int, default=8192)
    ap.add_argument("--chunk-size", type=int, default=512)
    ap.add_argument("--num-targets", type=int, default=512)
    ap.add_argument("--cache-name", default="h2o-torch-quantized8")
    ap.add_argument("--lora-r", type=int, default=16)
    ap.add_argument("--no-kv-offload", action="store_true")
    ap.add_argument("--n-layer", type=int, default=None, help="fewer layers (the result is then marked reduced)")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    args = ap.parse_args()
    from keys_values_b200 import ops
    from keys_values_b200.finetune.engine import build_lora_training_setup, training_step
    from keys_values_b200.ops import cuda as cu

    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = args.tp or world
    setup = build_lora_training_setup(
        args.model, dev, torch.bfloat16, cache_name=args.cache_name, cache_length=args.cache_length, chunk_size=args.chunk_size,
        lora_r=args.lora_r, lora_alpha=2 * args.lora_r, lora_targets=("query", "key", "value", "projection", "mlp"), micro_batch_size=1,
        n_layer=args.n_layer, world_size=world, rank=rank, seed=1234, tp_size=tp, kv_cpu_offload=not args.no_kv_offload,
    )
    vocab = setup.config.vocab_size
    replica = rank // tp
    gen = torch.Generator().manual_seed(99 + replica)  # the ranks of a replica see the same sequence
    total = args.warmup + args.steps
    host = [(torch.randint(0, vocab, (1, args.seq_len), generator=gen).pin_memory(),
             torch.randint(0, vocab, (1, args.num_targets), generator=gen).pin_memory()) for _ in range(total)]

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for k in range(args.warmup):
        training_step(setup, host[k][0].to(dev, non_blocking=True), host[k][1].to(dev, non_blocking=True))
    sync()
    launches0 = ops.native_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    losses = []
    for k in range(args.warmup, total):
        loss = training_step(setup, host[k][0].to(dev, non_blocking=True), host[k][1].to(dev, non_blocking=True))
        losses.append(float(loss.float().cpu()))
    e1.record()
    sync()
    cu.check_status(dev)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    if rank == 0:
        replicas = world // tp
        print(json.dumps({
            "bench": "long-context LoRA training step, tensor parallel",
            "model": args.model + (f" (REDUCED to {args.n_layer} layers)" if args.n_layer else ""), "n_gpus": world,
            "parallelism": f"dp{replicas} x tp{tp}", "seq_len": args.seq_len, "cache": args.cache_name, "cache_length": args.cache_length,
            "chunk_size": args.chunk_size, "lora": f"r={args.lora_r} on all linears", "kv_offload_to_host": not args.no_kv_offload,
            "steps": args.steps, "warmup": args.warmup, "s_per_step": ms / 1e3 / args.steps,
            "tokens_per_s": replicas * args.seq_len * args.steps / (ms / 1e3), "loss": losses[-1],
            "native_launches": ops.native_launches() - launches0, "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2**30,
        }), flush=True)
    if setup.extras.get("tp_comm") is not None:
        setup.gpt_model.close()
        setup.extras["tp_comm"].close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
