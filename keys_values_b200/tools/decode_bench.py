"""Prefill and decode throughput of chunked inference through a bounded KV cache, on one GPU or tensor
parallel over the GPUs of one node.

    python -m keys_values_b200.tools.decode_bench [--model Llama-3-8B] [--batch 4] [--prompt 65536] \
        [--decode 512] [--cache-name h2o-torch-quantized4] [--cache-length 8192] [--n-layer N]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m keys_values_b200.tools.decode_bench

Random-init weights of the named architecture, synthetic prompts. Under ``torch.distributed.run`` the model
is sharded over KV heads and MLP columns (:class:`keys_values_b200.parallel.tp.TPGPT`), one rank per GPU.
Prefill is timed as one chunked pass over the prompts (CUDA events, maximum over ranks); decode as
``--decode`` greedy single-token steps (replayed from a CUDA graph unless ``--no-graph``). Prints one JSON
line with prefill tokens/s and decode tokens/s (all batch rows together).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Optional

import torch


def run(model_name: str = "Llama-3-8B", batch: int = 4, prompt: int = 65536, decode: int = 512, cache_name: str = "h2o-torch-quantized4",
        cache_length: int = 8192, chunk_size: int = 2048, use_graph: bool = True, n_layer: Optional[int] = None,
        fused_prefill: Optional[bool] = None, warmup_decode: int = 8, repeats: int = 1) -> dict:
    """One measurement; returns the result record on rank 0 and ``{}`` elsewhere. The process group is set up
    (and torn down) here when the environment names more than one rank."""
    import torch.distributed as dist

    from keys_values_b200 import ops
    from keys_values_b200.config import Config
    from keys_values_b200.generate.base import _prefill, batched_sample
    from keys_values_b200.generate.decode_graph import Decoder
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.models.model import GPT
    from keys_values_b200.ops import cuda as cu

    rank, local_rank, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    own_group = world > 1 and not dist.is_initialized()
    if own_group:
        dist.init_process_group("nccl", device_id=dev)
    kw = {} if n_layer is None else dict(n_layer=n_layer)
    cfg = Config.from_name(model_name, **kw)
    torch.manual_seed(0)  # the same on every rank: replicated parameters (embedding, norms, head) must agree
    comm = None
    with torch.device(dev):
        if world > 1:
            from keys_values_b200.parallel.tp import TPComm, TPGPT

            comm = TPComm(world, rank, dev)
            model = TPGPT(cfg, comm, fused_prefill=fused_prefill).to(torch.bfloat16)
        else:
            model = GPT(cfg).to(torch.bfloat16)
    model.eval()
    model.assign_kv_caches(KVCacheFactory.create(model, cache_name, batch, cache_length, dtype=torch.bfloat16, device=dev,
                                                 cache_kwargs=dict(max_chunk_size=chunk_size)))
    gen = torch.Generator().manual_seed(7)
    host_prompts = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=gen).pin_memory()
    max_len = prompt + decode + warmup_decode + 8  # context width of the position encoding

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    greedy = dict(temperature=0.0)
    records = []
    with torch.inference_mode():
        # warm-up on a short prompt (kernel loading, allocator, symmetric buffers of the largest chunk)
        _prefill(model, host_prompts[:, : min(prompt, 2 * cache_length)].to(dev), chunk_size, max_len)
        for _ in range(repeats):
            sync()
            launches0 = ops.native_launches()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
            prompts = host_prompts.to(dev, non_blocking=True)  # the step's input arrives from pinned host memory
            logits = _prefill(model, prompts, chunk_size, max_len)
            e[1].record()
            tokens = logits.argmax(-1).view(batch, 1)
            decoder = Decoder(model, batch, use_graph=use_graph)
            for _ in range(warmup_decode):  # two eager steps, the capture, replays
                tokens = batched_sample(decoder(tokens)[:, -1:], greedy).view(batch, 1)
            sync()
            e[2].record()
            out_tokens = []
            for _ in range(decode):
                tokens = batched_sample(decoder(tokens)[:, -1:], greedy).view(batch, 1)
                out_tokens.append(tokens)
            host_tokens = torch.cat(out_tokens, dim=1).cpu()  # device→host read of the generated tokens
            e[3].record()
            sync()
            records.append((e[0].elapsed_time(e[1]) / 1e3, e[2].elapsed_time(e[3]) / 1e3, ops.native_launches() - launches0, host_tokens,
                            decoder))
    cu.check_status(dev)
    t_pre, t_dec, launches, host_tokens, decoder = min(records, key=lambda r: r[0] + r[1])
    same_tokens = True
    if world > 1:
        t = torch.tensor([t_pre, t_dec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_pre, t_dec = t.tolist()
        mine = host_tokens.to(dev)
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        same_tokens = all(torch.equal(o, mine) for o in everyone)
    result = {
        "bench": "chunked inference", "model": model_name + (f" (REDUCED to {n_layer} layers)" if n_layer else ""),
        "tp": world, "batch": batch, "prompt": prompt, "decode_steps": decode, "cache": cache_name, "cache_length": cache_length,
        "chunk_size": chunk_size, "prefill_path": ("fused all-gather/GEMM/reduce-scatter" if model.fused_prefill else "all-reduce") if world > 1 else "single GPU",
        "decode_mode": "cuda graph" if decoder.graph is not None else f"eager ({decoder.reason or 'requested'})",
        "prefill_tokens_per_s": batch * prompt / t_pre, "decode_tokens_per_s": batch * decode / t_dec,
        "ms_per_decode_step": 1e3 * t_dec / decode, "prefill_s": t_pre, "decode_s": t_dec,
        "total_tokens_per_s": batch * (prompt + decode) / (t_pre + t_dec),
        "native_launches": launches, "ranks_generated_same_tokens": same_tokens,
        "h2d_bytes": host_prompts.numel() * host_prompts.element_size(), "d2h_bytes": host_tokens.numel() * host_tokens.element_size(),
        "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2**30,
    }
    if comm is not None:
        model.close()
        comm.close()
    if own_group:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Llama-3-8B")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=65536)
    ap.add_argument("--decode", type=int, default=512)
    ap.add_argument("--cache-name", default="h2o-torch-quantized4")
    ap.add_argument("--cache-length", type=int, default=8192)
    ap.add_argument("--chunk-size", type=int, default=2048)
    ap.add_argument("--no-graph", action="store_true", help="eager single-token steps instead of CUDA graph replays")
    ap.add_argument("--no-fused-prefill", action="store_true", help="tensor parallel: all-reduce path for the prefill chunks too")
    ap.add_argument("--fused-prefill", action="store_true", help="tensor parallel: fused path below 8 ranks too (default: from 8 ranks on)")
    ap.add_argument("--n-layer", type=int, default=None, help="fewer layers (the result is then marked reduced)")
    ap.add_argument("--repeats", type=int, default=1)
    args = ap.parse_args()
    out = run(args.model, args.batch, args.prompt, args.decode, args.cache_name, args.cache_length, args.chunk_size, not args.no_graph,
              args.n_layer, False if args.no_fused_prefill else (True if args.fused_prefill else None), repeats=args.repeats)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
