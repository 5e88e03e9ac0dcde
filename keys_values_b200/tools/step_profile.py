"""Which kernels a long-context training step spends its GPU time in.

    python -m keys_values_b200.tools.step_profile [--n-layer 4] [--model Qwen3-4B] [--seq-len 131072] [--top 30]

Runs the flagship LoRA step (H2O int8 cache of 16384 slots, chunks of 1024) on a model cut to ``--n-layer`` layers:
two warm-up steps, one step timed without any profiler (CUDA events), then one step under the PyTorch profiler,
whose kernel times are reported as SHARES of the step's device time (absolute times under a profiler are not
benchmark numbers). The per-layer shares carry over to the full model: every layer runs the same kernels.
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen3-4B")
    ap.add_argument("--n-layer", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=131072)
    ap.add_argument("--cache-length", type=int, default=16384)
    ap.add_argument("--chunk-size", type=int, default=1024)
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--ops", action="store_true", help="a second table: device time per framework operator (aten::* and the native ops)")
    args = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile

    from keys_values_b200.finetune.engine import build_lora_training_setup, training_step

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    setup = build_lora_training_setup(model_name=args.model, device=dev, dtype=torch.bfloat16, cache_name="h2o-torch-quantized8",
                                      cache_length=args.cache_length, chunk_size=args.chunk_size, lora_r=8, lora_alpha=16,
                                      lora_targets=("query", "key", "value", "projection"), micro_batch_size=1, n_layer=args.n_layer,
                                      yarn_rope=True, seed=1234)
    vocab = setup.config.vocab_size
    ids = torch.randint(0, vocab, (1, args.seq_len), device=dev)
    tg = torch.randint(0, vocab, (1, args.chunk_size), device=dev)
    for _ in range(2):
        training_step(setup, ids, tg)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    training_step(setup, ids, tg)
    e1.record()
    torch.cuda.synchronize(dev)
    print(f"step of {args.n_layer} layers, {args.seq_len} tokens: {e0.elapsed_time(e1) / 1e3:.3f} s (CUDA events, no profiler)")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        training_step(setup, ids, tg)
        torch.cuda.synchronize(dev)
    rows = sorted(((e.device_time_total, e.count, e.key) for e in prof.key_averages() if e.device_time_total > 0), reverse=True)
    total = sum(r[0] for r in rows)
    print(f"{'share':>7} {'calls':>7}  kernel")
    for t, c, k in rows[: args.top]:
        print(f"{100 * t / total:6.1f}% {c:7d}  {k[:120]}")
    rest = sum(r[0] for r in rows[args.top:])
    print(f"{100 * rest / total:6.1f}% {sum(r[1] for r in rows[args.top:]):7d}  ({len(rows) - args.top} more kernels)")
    if args.ops:
        # which framework operators launch the small kernels: one more step with the host side recorded as well
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
            training_step(setup, ids, tg)
            torch.cuda.synchronize(dev)
        ops = sorted(((e.self_device_time_total, e.count, e.key, str(e.input_shapes)[:90]) for e in prof.key_averages(group_by_input_shape=True)
                      if e.self_device_time_total > 0 and e.key.startswith("aten::")), reverse=True)
        print(f"{'share':>7} {'calls':>7}  operator (input shapes)")
        for t, c, k, shp in ops[: args.top]:
            print(f"{100 * t / total:6.1f}% {c:7d}  {k} {shp}")


if __name__ == "__main__":
    main()
