"""Throughput of chunked inference for every cache policy and buffer type
(``keys_values/scripts/profile_caches.py``).

    python -m keys_values_b200.tools.profile_caches [--model tiny-qwen3] [--seq-len 4096] [--cache-length 1024] [--chunk-size 256]

For each cache name a random-init model of the named architecture processes one batch of random
tokens; printed: tokens/s (CUDA events on a GPU, wall clock on a CPU) and peak memory.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def profile(model_name: str, cache_names, batch: int, seq_len: int, cache_length: int, chunk_size: int, device, dtype, n_layer=None):
    from keys_values_b200.config import Config
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.long_context import LongContextInferenceModel
    from keys_values_b200.models.head_model import CrossEntropyOnLogits
    from keys_values_b200.models.model import GPT

    cfg = Config.from_name(model_name, **({} if n_layer is None else dict(n_layer=n_layer)))
    torch.manual_seed(0)
    with torch.device(device):
        model = GPT(cfg).to(dtype)
    model.eval()
    ids = torch.randint(0, cfg.vocab_size, (batch, seq_len), device=device)
    rows = []
    for name in cache_names:
        try:
            kw = dict(max_chunk_size=chunk_size) if not name.startswith(("dense", "lastrec", "smart")) else {}
            length = seq_len if name.startswith("dense") else cache_length
            model.assign_kv_caches(KVCacheFactory.create(model, name, batch, length, dtype=dtype, device=device, cache_kwargs=kw))
            lcm = LongContextInferenceModel(model, CrossEntropyOnLogits(cfg), chunk_size=chunk_size)
            times = []
            for _ in range(2):  # the second pass is the one reported
                model.reset()
                if device.type == "cuda":
                    torch.cuda.reset_peak_memory_stats(device)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                t0 = time.perf_counter()
                with torch.inference_mode():
                    lcm(ids, None)
                if device.type == "cuda":
                    e1.record()
                    torch.cuda.synchronize(device)
                    times.append(e0.elapsed_time(e1) / 1e3)
                else:
                    times.append(time.perf_counter() - t0)
            rows.append({"cache": name, "tokens_per_s": batch * seq_len / times[-1], "seconds": times[-1],
                         "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30 if device.type == "cuda" else None})
        except Exception as ex:  # a cache that the configuration does not support is reported, not fatal
            rows.append({"cache": name, "error": f"{type(ex).__name__}: {ex}"[:200]})
        finally:
            model.clear_kv_caches()
    return rows


def main(argv=None) -> None:
    from keys_values_b200.kvcache.factory import KVCacheFactory

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-qwen3")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--cache-length", type=int, default=1024)
    ap.add_argument("--chunk-size", type=int, default=256)
    ap.add_argument("--n-layer", type=int, default=None)
    ap.add_argument("--caches", nargs="*", default=None)
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    names = a.caches or [n for n in KVCacheFactory.supported_names() if "bnb" not in n]
    for row in profile(a.model, names, a.batch, a.seq_len, a.cache_length, a.chunk_size, dev, dtype, a.n_layer):
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
