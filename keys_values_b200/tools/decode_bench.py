"""Prefill and decode throughput of chunked inference through a bounded KV cache.

    python -m keys_values_b200.tools.decode_bench [--model Llama-3-8B] [--batch 4] [--prompt 65536] \
        [--decode 512] [--cache-name h2o-torch-quantized4] [--cache-length 16384] [--n-layer N]

Random-init weights of the named architecture, synthetic prompts. Prefill is timed as one chunked
pass over the prompts (CUDA events); decode as ``--decode`` greedy single-token steps (replayed from a
CUDA graph unless ``--no-graph``). Prints one JSON
line with prefill tokens/s and decode tokens/s (all batch rows together).
"""
from __future__ import annotations

import argparse
import json

import torch

from keys_values_b200.config import Config
from keys_values_b200.generate.base import _prefill, batched_sample
from keys_values_b200.generate.decode_graph import Decoder
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.models.model import GPT


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Llama-3-8B")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=65536)
    ap.add_argument("--decode", type=int, default=512)
    ap.add_argument("--cache-name", default="h2o-torch-quantized4")
    ap.add_argument("--cache-length", type=int, default=16384)
    ap.add_argument("--chunk-size", type=int, default=2048)
    ap.add_argument("--no-graph", action="store_true", help="eager single-token steps instead of CUDA graph replays")
    ap.add_argument("--n-layer", type=int, default=None, help="fewer layers (the result is then marked reduced)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    kw = {} if args.n_layer is None else dict(n_layer=args.n_layer)
    cfg = Config.from_name(args.model, **kw)
    torch.manual_seed(0)
    with torch.device(dev):
        model = GPT(cfg).to(torch.bfloat16)
    model.eval()
    caches = KVCacheFactory.create(model, args.cache_name, args.batch, args.cache_length, dtype=torch.bfloat16, device=dev,
                                   cache_kwargs=dict(max_chunk_size=args.chunk_size))
    model.assign_kv_caches(caches)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), device=dev)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    max_len = args.prompt + args.decode + 16  # context width of the position encoding: prompt + warm-up + timed steps
    with torch.inference_mode():
        # warm-up on a short prompt (kernel loading, allocator)
        _prefill(model, prompts[:, : min(args.prompt, 2 * args.cache_length)], args.chunk_size, max_len)
        torch.cuda.synchronize()
        e[0].record()
        logits = _prefill(model, prompts, args.chunk_size, max_len)
        e[1].record()
        tokens = logits.argmax(-1).view(args.batch, 1)
        decoder = Decoder(model, args.batch, use_graph=not args.no_graph)
        greedy = dict(temperature=0.0)
        for _ in range(8):  # two eager steps, the capture, five replays
            tokens = batched_sample(decoder(tokens)[:, -1:], greedy).view(args.batch, 1)
        torch.cuda.synchronize()
        e[2].record()
        for _ in range(args.decode):
            tokens = batched_sample(decoder(tokens)[:, -1:], greedy).view(args.batch, 1)
        e[3].record()
        torch.cuda.synchronize()
    from keys_values_b200.ops import cuda as cu

    cu.check_status(dev)
    t_pre, t_dec = e[0].elapsed_time(e[1]) / 1e3, e[2].elapsed_time(e[3]) / 1e3
    print(json.dumps({
        "bench": "chunked inference", "model": args.model + (f" (REDUCED to {args.n_layer} layers)" if args.n_layer else ""),
        "batch": args.batch, "prompt": args.prompt, "decode_steps": args.decode, "cache": args.cache_name,
        "cache_length": args.cache_length,
        "decode_mode": "cuda graph" if decoder.graph is not None else f"eager ({decoder.reason or 'requested'})", "prefill_tokens_per_s": args.batch * args.prompt / t_pre,
        "decode_tokens_per_s": args.batch * args.decode / t_dec, "ms_per_decode_step": 1e3 * t_dec / args.decode,
        "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2**30,
    }), flush=True)


if __name__ == "__main__":
    main()
