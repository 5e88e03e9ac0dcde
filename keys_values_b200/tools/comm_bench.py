"""Device-timed benchmark of the fused compute+collective kernels against NCCL + library GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 -m keys_values_b200.tools.comm_bench [--out file.jsonl]

One process per GPU. Every number is the median over iterations of CUDA-event times on the
launching stream, maximised over ranks. The roofline of a fused kernel is the slower of
(FLOPs / measured library GEMM peak) and (bytes that cross NVLink per GPU / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0  # measured peer copy, per direction per GPU


def _timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default="all", choices=["all", "oneshot", "allreduce", "tp_gemm"])
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.parallel.symm import SymmetricArena
    from keys_values_b200.parallel.tp import TPContext

    peaks = {"bf16_tflops": 1619.7}
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        peaks.update({k: v for k, v in json.loads(p.read_text()).items() if k in peaks})
    fh = open(args.out, "a") if (args.out and rank == 0) else None

    def out(d):
        if rank == 0:
            line = json.dumps(d)
            print(line, flush=True)
            if fh:
                fh.write(line + "\n")
                fh.flush()

    # ------------------------------------------- one-shot all-reduce (decode steps under tensor parallelism)
    if args.only in ("all", "oneshot"):
        from keys_values_b200.parallel.tp import TPComm

        comm = TPComm(world, rank, dev)
        K = 64  # all-reduces per graph: a decode step of a 32-layer model has 64
        for rows, feat in ((4, 4096), (16, 4096), (32, 4096)):
            src = torch.randn(rows, feat, device=dev, dtype=torch.bfloat16)
            res = torch.randn(rows, feat, device=dev, dtype=torch.bfloat16)
            ref = src.clone()
            outs = []

            def fused():
                for _ in range(K):
                    buf = comm.out_buffer(rows, feat, torch.bfloat16)
                    buf.copy_(src)  # stands for the producer GEMM that writes into symmetric memory
                    outs.append(comm.all_reduce(buf, residual=res))
                    outs.clear()

            def lib():
                for _ in range(K):
                    ref.copy_(src)
                    dist.all_reduce(ref)
                    torch.add(ref, res)

            # both as CUDA graphs (as in the captured decode step): device time without the host's launch cost
            fused(), lib()
            torch.cuda.synchronize()
            g_f, g_n = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_f):
                comm.begin_capture()
                fused()
                comm.end_capture()
            with torch.cuda.graph(g_n):
                lib()
            ms_f, ms_n = _timed(g_f.replay) / K, _timed(g_n.replay) / K
            cu.check_status(dev)
            out({"bench": "oneshot_allreduce_bf16_plus_residual", "world": world, "rows": rows, "features": feat, "bytes": rows * feat * 2,
                 "calls_per_graph": K, "fused_us_per_call": ms_f * 1e3, "nccl_plus_add_us_per_call": ms_n * 1e3,
                 "note": "each call includes a copy of the payload (the producer's write); graph replay, max over ranks"})
            del g_f, g_n  # the graphs hold communicator work: gone before the buffers and the process group are
            torch.cuda.synchronize()
        comm.close()

    # ---------------------------------------------------------------- all-reduce (gradient mean)
    for mib in ((16, 128, 1024) if args.only in ("all", "allreduce") else ()):
        n = mib * 2**20 // 2
        arena = SymmetricArena(n, torch.bfloat16, dev, world, rank)
        arena.tensor.normal_()
        ref = arena.tensor.clone()
        ms_f = _timed(lambda: arena.all_reduce_mean_(0, n))
        ms_n = _timed(lambda: dist.all_reduce(ref))
        cu.check_status(dev)
        bus = 2.0 * (world - 1) / world * n * 2 / 1e9
        out({"bench": "allreduce_mean_bf16", "world": world, "MiB": mib, "fused_us": ms_f * 1e3, "nccl_us": ms_n * 1e3,
             "fused_busbw_gbs": bus / (ms_f / 1e3), "nccl_busbw_gbs": bus / (ms_n / 1e3),
             "fused_frac_of_nvlink": bus / (ms_f / 1e3) / NVLINK_GBS})
        arena.close()

    # ------------------------------------------- all-gather -> GEMM and GEMM -> reduce-scatter
    # token-parallel rows of a cell of the flagship model (n_embd 2560, MLP 9728, QKV 6144)
    for rows, K, N in (((2048, 2560, 6144), (2048, 2560, 9728), (4096, 2560, 9728)) if args.only in ("all", "tp_gemm") else ()):
        M = world * rows
        ctx = TPContext(world, rank, dev, max_rows=M, max_features=max(K, N))
        shard = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        ctx.stage_view(rows, K).copy_(shard)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

        def lib_ag():
            dist.all_gather_into_tensor(full, shard)
            torch.matmul(full, w.t(), out=o)

        ms_f = _timed(lambda: ctx.allgather_gemm(rows, w, out=o))
        ms_l = _timed(lib_ag)
        cu.check_status(dev)
        flops = 2.0 * M * N * K
        nv_bytes = (world - 1) * rows * K * 2
        roof = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (NVLINK_GBS * 1e9))
        out({"bench": "allgather_gemm", "world": world, "M": M, "N": N, "K": K, "fused_us": ms_f * 1e3, "nccl_cublas_us": ms_l * 1e3,
             "fused_tflops": flops / ms_f / 1e9, "roofline_us": roof * 1e6, "frac_of_roofline": roof / (ms_f / 1e3)})

        # GEMM -> reduce-scatter: x (M, K/world shard), weight (N, K/world)
        Ks = N // world // 64 * 64  # reuse N as the contracted dimension (down projection)
        x = torch.randn(M, Ks, device=dev, dtype=torch.bfloat16)
        w2 = torch.randn(K, Ks, device=dev, dtype=torch.bfloat16) * 0.02
        part = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        rs = torch.empty(rows, K, device=dev, dtype=torch.bfloat16)

        def lib_rs():
            torch.matmul(x, w2.t(), out=part)
            dist.reduce_scatter_tensor(rs, part)

        ms_f = _timed(lambda: ctx.gemm_reduce_scatter(x, w2, out=rs))
        ms_l = _timed(lib_rs)
        cu.check_status(dev)
        flops = 2.0 * M * K * Ks
        nv_bytes = (world - 1) * rows * K * 2
        roof = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (NVLINK_GBS * 1e9))
        out({"bench": "gemm_reduce_scatter", "world": world, "M": M, "N": K, "K": Ks, "fused_us": ms_f * 1e3,
             "cublas_nccl_us": ms_l * 1e3, "fused_tflops": flops / ms_f / 1e9, "roofline_us": roof * 1e6,
             "frac_of_roofline": roof / (ms_f / 1e3)})
        ctx.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
