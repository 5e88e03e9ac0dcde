"""Kernel-level reference arm: the reference's own SDPA-with-summed-weights path, timed on the grid that
``keys_values_b200.tools.microbench sdpa`` times for this framework.

    python baseline/reference_kernels.py [--out file.jsonl]

The call is the reference's public one, ``FlashInferSDPA.scaled_dot_product_attention(..., return_attn_weights=True)``
(``keys_values/attention/flashinfer_wrapper.py:367``): its FlashInfer-derived prefill / decode kernels (unchanged
sources rebuilt for compute_100 by ``baseline/install_reference.py``) followed by its Triton score-sum kernel, and,
where slot order is not position order, its key/value reordering. Nothing of ``keys_values_b200`` is imported here.
Same shapes, same data, same timing rules (CUDA events after warm-up, L2 flushed between iterations).
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def time_fn(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    for p in (str(HERE / "shim"), str(HERE / "_ref")):
        if p not in sys.path:
            sys.path.insert(0, p)
    fh = open(args.out, "a") if args.out else None

    def out(d):
        d["impl"] = "reference"
        line = json.dumps(d)
        print(line, flush=True)
        if fh:
            fh.write(line + "\n")
            fh.flush()

    try:
        wrapper = importlib.import_module("keys_values.attention.flashinfer_wrapper")
        sdpa = wrapper.FlashInferSDPA()
    except Exception as ex:
        out({"unavailable": f"{type(ex).__name__}: {str(ex)[:200]}"})
        return
    dev = torch.device("cuda")
    flush = torch.empty(192 * 2**20, dtype=torch.uint8, device=dev)
    H, G, D = 32, 8, 128
    scale = 1 / math.sqrt(D)
    cases = [(B, q, kv, False) for B in (1, 4) for q in (1, 256, 2048) for kv in (4096, 16384, 32768)]
    cases += [(1, 1024, 16384, True), (4, 1024, 16384, True)]  # a training chunk: slots in random order
    for B, q_len, kv, scattered in cases:
        g = torch.Generator(device=dev).manual_seed(0)
        q = torch.randn(B, H, q_len, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
        k = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
        v = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
        input_pos = kv - q_len if not scattered else 4 * kv
        token_pos = None
        if scattered:
            # the cache holds kv of the input_pos + q_len tokens seen so far, the new chunk among them, in random slots
            rows = []
            for _ in range(B * G):
                old = torch.randperm(input_pos, device=dev, generator=g)[: kv - q_len]
                new = torch.arange(input_pos, input_pos + q_len, device=dev)
                both = torch.cat((old, new))
                rows.append(both[torch.randperm(kv, device=dev, generator=g)])
            token_pos = torch.stack(rows).view(B, G, kv).to(torch.int32)
        fn = lambda: sdpa.scaled_dot_product_attention(q, k, v, scale, input_pos, token_pos, return_attn_weights=True)  # noqa: E731
        try:
            ms = time_fn(fn, flush=flush)
        except Exception as ex:
            out({"bench": "sdpa_w", "B": B, "q": q_len, "kv": kv, "scattered": scattered, "error": f"{type(ex).__name__}: {str(ex)[:200]}"})
            continue
        out({"bench": "sdpa_w", "B": B, "q": q_len, "kv": kv, "scattered": scattered, "us": ms * 1e3})


if __name__ == "__main__":
    main()
