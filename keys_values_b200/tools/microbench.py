"""Kernel micro-benchmarks: CUDA-event timing after warm-up, with an L2 flush
(a write larger than the 126 MB L2) between timed iterations.

    python -m keys_values_b200.tools.microbench sdpa|sdpa_train|sdpa_bwd|sdpa_variants|sdpa_head_sizes|gemm|elementwise|all [--out file.jsonl]

``sdpa`` covers the SDPA-with-weights grid: bf16 GQA 32/8 heads, head size 128,
batch 1 and 4, query length {1, 256, 2048}, KV length {4096, 16384, 32768}.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def _flush_buf(dev):
    return torch.empty(192 * 2**20, dtype=torch.uint8, device=dev)


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


def bench_sdpa(out, peaks):
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    H, G, D = 32, 8, 128
    scale = 1 / math.sqrt(D)
    for B in (1, 4):
        for q_len in (1, 256, 2048):
            for kv in (4096, 16384, 32768):
                g = torch.Generator(device=dev).manual_seed(0)
                q = torch.randn(B, H, q_len, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
                k = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
                v = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16, generator=g) * scale
                input_pos = kv - q_len
                if q_len == 1:
                    from keys_values_b200 import ops

                    fn = lambda: ops.decode_attention(q, k, v, scale, input_pos, None, True)  # noqa: E731
                else:
                    fn = lambda: cu.sdpa_fwd(q, k, v, scale, input_pos, None, True)  # noqa: E731
                try:
                    ms = time_fn(fn, flush=flush)
                except Exception as ex:  # pragma: no cover
                    out({"bench": "sdpa_w", "B": B, "q": q_len, "kv": kv, "error": str(ex)})
                    continue
                cu.check_status(dev)
                # useful work: QK^T and PV over the causally visible part
                vis = kv - q_len / 2 if q_len > 1 else kv
                flops = 4.0 * B * H * q_len * vis * D
                bytes_ = 2.0 * (2 * B * G * kv * D + 2 * B * H * q_len * D) + 4.0 * B * G * kv
                t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), bytes_ / (peaks["hbm_gbs"] * 1e9))
                out({"bench": "sdpa_w", "B": B, "q": q_len, "kv": kv, "us": ms * 1e3, "tflops": flops / ms / 1e9,
                     "frac_of_measured_roofline": t_roof / (ms / 1e3)})


def bench_sdpa_bwd(out, peaks):
    """Backward (dQ launch + dK/dV launch + delta kernel) on the training-chunk shapes: a chunk of
    ``q`` new tokens against a cache of ``kv`` slots in random slot order."""
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    H, G, D = 32, 8, 128
    scale = 1 / math.sqrt(D)
    for B, q_len, kv in ((1, 1024, 16384), (1, 2048, 16384), (4, 1024, 16384), (1, 16384, 16384)):
        q = torch.randn(B, H, q_len, D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, G, kv, D, device=dev, dtype=torch.bfloat16)
        if q_len < kv:
            tp = torch.stack([torch.stack([torch.randperm(kv, device=dev) for _ in range(G)]) for _ in range(B)]).to(torch.int32)
            tp[:, :, :q_len] = (torch.arange(q_len, device=dev) + 2 * kv).to(torch.int32)
            input_pos = 2 * kv
        else:
            tp, input_pos = None, 0
        o, _, lse = cu.sdpa_fwd(q, k, v, scale, input_pos, tp, False)
        go = torch.randn_like(o)
        dk = torch.zeros(B, G, kv, D, device=dev)
        dv = torch.zeros_like(dk)
        ms = time_fn(lambda: cu.sdpa_bwd(go, q, k, v, o, lse, scale, input_pos, tp, dk, dv), flush=flush)
        cu.check_status(dev)
        vis = kv - q_len / 2
        flops = 10.0 * B * H * q_len * vis * D  # five GEMMs of useful work
        out({"bench": "sdpa_bwd", "B": B, "q": q_len, "kv": kv, "us": ms * 1e3, "tflops": flops / ms / 1e9,
             "frac_of_measured_peak": flops / ms / 1e9 / peaks["bf16_tflops"]})


def bench_sdpa_train(out, peaks):
    """The attention calls of one (layer, chunk) of the training step: ``q`` new tokens whose K/V sit
    in random slots of a full cache of ``kv`` slots (an evicting cache), forward with weights and
    backward."""
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    H, G, D = 32, 8, 128
    scale = 1 / math.sqrt(D)
    for B, T, L in ((1, 1024, 16384), (1, 2048, 16384), (4, 1024, 16384)):
        q = torch.randn(B, H, T, D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        tp = torch.stack([torch.stack([torch.randperm(L, device=dev) for _ in range(G)]) for _ in range(B)]).to(torch.int32)
        newslots = torch.randperm(L, device=dev)[:T]
        tp[:, :, newslots] = (torch.arange(T, device=dev) + 2 * L).to(torch.int32)
        ip = 2 * L
        ms_f = time_fn(lambda: cu.sdpa_fwd(q, k, v, scale, ip, tp, True), flush=flush)
        o, _, lse = cu.sdpa_fwd(q, k, v, scale, ip, tp, False)
        go = torch.randn_like(o)
        dk = torch.zeros(B, G, L, D, device=dev)
        dv = torch.zeros_like(dk)
        ms_b = time_fn(lambda: cu.sdpa_bwd(go, q, k, v, o, lse, scale, ip, tp, dk, dv), flush=flush)
        cu.check_status(dev)
        flops = 4.0 * B * H * T * L * D
        out({"bench": "sdpa_train_chunk", "B": B, "q": T, "kv": L, "fwd_us": ms_f * 1e3, "bwd_us": ms_b * 1e3,
             "fwd_tflops": flops / ms_f / 1e9, "bwd_tflops": 2.5 * flops / ms_b / 1e9,
             "fwd_frac_of_measured_peak": flops / ms_f / 1e9 / peaks["bf16_tflops"],
             "bwd_frac_of_measured_peak": 2.5 * flops / ms_b / 1e9 / peaks["bf16_tflops"]})


def bench_sdpa_variants(out, peaks):
    """Sliding window and logit soft-capping on the training chunk (plain prefix positions): forward with summed
    weights and backward with accumulation."""
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    B, H, G, D, T, L = 1, 32, 8, 128, 1024, 16384
    scale = 1 / math.sqrt(D)
    q = torch.randn(B, H, T, D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
    go = torch.randn(B, T, H * D, device=dev, dtype=torch.bfloat16)
    dk = torch.zeros(B, G, L, D, device=dev)
    dv = torch.zeros_like(dk)
    ip = L - T
    for window, softcap in ((None, None), (4096, None), (None, 50.0), (4096, 50.0)):
        ms_f = time_fn(lambda: cu.sdpa_fwd(q, k, v, scale, ip, None, True, window, softcap), flush=flush)
        o, _, lse = cu.sdpa_fwd(q, k, v, scale, ip, None, False, window, softcap)
        ms_b = time_fn(lambda: cu.sdpa_bwd(go, q, k, v, o, lse, scale, ip, None, dk, dv, window, softcap), flush=flush)
        cu.check_status(dev)
        out({"bench": "sdpa_variants", "B": B, "q": T, "kv": L, "window": window, "softcap": softcap,
             "fwd_with_weights_us": ms_f * 1e3, "bwd_us": ms_b * 1e3})


def bench_sdpa_head_sizes(out, peaks):
    """Forward with summed weights on the training chunk for the head sizes the kernels cover (256: forward only)."""
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    B, T, L = 1, 1024, 16384
    for D, H, G in ((64, 32, 8), (128, 32, 8), (256, 16, 8)):
        scale = 1 / math.sqrt(D)
        q = torch.randn(B, H, T, D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        ms_w = time_fn(lambda: cu.sdpa_fwd(q, k, v, scale, L - T, None, True), flush=flush)
        ms = time_fn(lambda: cu.sdpa_fwd(q, k, v, scale, L - T, None, False), flush=flush)
        cu.check_status(dev)
        flops = 4.0 * B * H * T * L * D
        out({"bench": "sdpa_head_size", "D": D, "H": H, "G": G, "q": T, "kv": L, "fwd_with_weights_us": ms_w * 1e3, "fwd_us": ms * 1e3,
             "fwd_tflops": flops / ms / 1e9, "fwd_frac_of_measured_peak": flops / ms / 1e9 / peaks["bf16_tflops"]})


def bench_gemm(out, peaks):
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    shapes = [(12288, 6144, 2560), (12288, 2560, 4096), (12288, 9728, 2560), (12288, 2560, 9728), (1024, 6144, 2560),
              (8192, 8192, 8192), (16384, 6144, 2560)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        ms = time_fn(lambda: cu.gemm(a, b), flush=flush)
        cu.check_status(dev)
        ms_pair = time_fn(lambda: cu.gemm_pair(a, b), flush=flush)
        cu.check_status(dev)
        ms_ref = time_fn(lambda: torch.matmul(a, b.t()), flush=flush)
        fl = 2.0 * M * N * K
        out({"bench": "gemm_bf16", "M": M, "N": N, "K": K, "us": ms * 1e3, "tflops": fl / ms / 1e9,
             "pair_us": ms_pair * 1e3, "pair_tflops": fl / ms_pair / 1e9,
             "cublas_us": ms_ref * 1e3, "cublas_tflops": fl / ms_ref / 1e9,
             "frac_of_measured_peak": fl / ms / 1e9 / peaks["bf16_tflops"],
             "pair_frac_of_measured_peak": fl / ms_pair / 1e9 / peaks["bf16_tflops"], "pair_over_cublas": ms_ref / ms_pair})


def bench_elementwise(out, peaks):
    from keys_values_b200 import ops

    dev = torch.device("cuda")
    flush = _flush_buf(dev)
    x = torch.randn(65536, 2560, device=dev, dtype=torch.bfloat16)
    w = torch.ones(2560, device=dev, dtype=torch.bfloat16)
    ms = time_fn(lambda: ops.rmsnorm(x, w, 1e-6), flush=flush)
    out({"bench": "rmsnorm_fwd", "GBps": 2 * x.numel() * 2 / ms / 1e6, "frac_of_measured_hbm": 2 * x.numel() * 2 / ms / 1e6 / peaks["hbm_gbs"]})
    a = torch.randn(32768, 9728, device=dev, dtype=torch.bfloat16)
    b = torch.randn_like(a)
    ms = time_fn(lambda: ops.swiglu(a, b), flush=flush)
    out({"bench": "swiglu_fwd", "GBps": 3 * a.numel() * 2 / ms / 1e6, "frac_of_measured_hbm": 3 * a.numel() * 2 / ms / 1e6 / peaks["hbm_gbs"]})
    T = 32768
    qkv = torch.randn(1, T, 48 * 128, device=dev, dtype=torch.bfloat16)
    cos = torch.randn(T, 128, device=dev)
    sin = torch.randn(T, 128, device=dev)
    ms = time_fn(lambda: ops.qknorm_rope(qkv, 32, 8, 128, cos, sin, w[:128], w[:128], 1e-6, 128), flush=flush)
    out({"bench": "qknorm_rope_fwd", "GBps": 2 * qkv.numel() * 2 / ms / 1e6, "frac_of_measured_hbm": 2 * qkv.numel() * 2 / ms / 1e6 / peaks["hbm_gbs"]})
    kv = torch.randn(4, 8, 16384, 128, device=dev, dtype=torch.bfloat16)
    ms = time_fn(lambda: ops.quantize_rows(kv, 8), flush=flush)
    out({"bench": "quantize_rows_int8", "GBps": kv.numel() * 3 / ms / 1e6, "frac_of_measured_hbm": kv.numel() * 3 / ms / 1e6 / peaks["hbm_gbs"]})
    sc = torch.rand(4, 8, 16384, device=dev)
    ww = torch.rand(4, 8, 16384, device=dev)
    ms = time_fn(lambda: ops.h2o_update(sc, ww, 1024, 16384), flush=flush)
    out({"bench": "h2o_update_C16384_k1024", "us": ms * 1e3})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    peaks = {"bf16_tflops": 1619.7, "hbm_gbs": 6548.5}
    try:
        from pathlib import Path

        p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
        if p.exists():
            peaks.update({k: v for k, v in json.loads(p.read_text()).items() if k in peaks})
    except Exception:
        pass
    fh = open(args.out, "a") if args.out else None

    def out(d):
        line = json.dumps(d)
        print(line, flush=True)
        if fh:
            fh.write(line + "\n")
            fh.flush()

    if args.which in ("gemm", "all"):
        bench_gemm(out, peaks)
    if args.which in ("sdpa", "all"):
        bench_sdpa(out, peaks)
    if args.which in ("sdpa_train", "all"):
        bench_sdpa_train(out, peaks)
    if args.which in ("sdpa_bwd", "all"):
        bench_sdpa_bwd(out, peaks)
    if args.which in ("sdpa_variants", "all"):
        bench_sdpa_variants(out, peaks)
    if args.which in ("sdpa_head_sizes", "all"):
        bench_sdpa_head_sizes(out, peaks)
    if args.which in ("elementwise", "all"):
        bench_elementwise(out, peaks)


if __name__ == "__main__":
    main()
