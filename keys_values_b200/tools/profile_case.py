"""Runs ONE small case of one kernel family, for use under ``ncu`` (a few launches, a few
hundred MB on the device). Inputs are larger than the 126 MB L2 only where stated.

    python -m keys_values_b200.tools.profile_case sdpa_fwd|sdpa_bwd|gemm|gemm_pair|decode|allreduce [--iters N]
"""
import argparse
import math

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--q", type=int, default=1024)
    ap.add_argument("--kv", type=int, default=16384)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--bits", type=int, default=8, help="decode: 16 (bf16 cache), 8 or 4")
    ap.add_argument("--head-size", type=int, default=128, help="sdpa_fwd: 128, 64 or 256 (256: 16 heads over 8 groups)")
    args = ap.parse_args()
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda")
    H, G, D = 32, 8, 128
    if args.which == "sdpa_fwd" and args.head_size != 128:
        D = args.head_size
        H = 16 if D == 256 else 32
    scale = 1 / math.sqrt(D)
    B, T, L = args.batch, args.q, args.kv
    torch.manual_seed(0)
    if args.which in ("sdpa_fwd", "sdpa_bwd"):
        q = torch.randn(B, H, T, D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, G, L, D, device=dev, dtype=torch.bfloat16)
        # an evicting cache in training: old tokens everywhere, the T tokens of the current chunk scattered over the slots
        input_pos = 6 * L
        tp = torch.empty(B, G, L, device=dev, dtype=torch.int32)
        for b in range(B):
            for g in range(G):
                old = torch.randperm(input_pos, device=dev)[: L - T]
                new = torch.arange(input_pos, input_pos + T, device=dev)
                tp[b, g] = torch.cat((old, new))[torch.randperm(L, device=dev)].to(torch.int32)
        if args.which == "sdpa_fwd":
            for _ in range(args.iters):
                out, w, lse = cu.sdpa_fwd(q, k, v, scale, input_pos, tp, True)
        else:
            out, w, lse = cu.sdpa_fwd(q, k, v, scale, input_pos, tp, False)
            go = torch.randn_like(out)
            dk = torch.zeros(B, G, L, D, device=dev)
            dv = torch.zeros_like(dk)
            for _ in range(args.iters):
                cu.sdpa_bwd(go, q, k, v, out, lse, scale, input_pos, tp, dk, dv)
    elif args.which == "gemm":
        a = torch.randn(12288, 2560, device=dev, dtype=torch.bfloat16)
        b = torch.randn(6144, 2560, device=dev, dtype=torch.bfloat16)
        for _ in range(args.iters):
            cu.gemm(a, b)
    elif args.which == "gemm_pair":
        a = torch.randn(12288, 2560, device=dev, dtype=torch.bfloat16)
        b = torch.randn(6144, 2560, device=dev, dtype=torch.bfloat16)
        for _ in range(args.iters):
            cu.gemm_pair(a, b)
    elif args.which == "decode":
        Bd = max(args.batch, 4)
        q = torch.randn(Bd, H, 1, D, device=dev, dtype=torch.bfloat16)
        if args.bits == 16:
            k = torch.randn(Bd, G, L, D, device=dev, dtype=torch.bfloat16)
            v = torch.randn_like(k)
            for _ in range(args.iters):
                cu.decode_attention(q, k, v, scale, L, True)
        else:
            Dq = D if args.bits == 8 else D // 2
            k = torch.randint(0, 255, (Bd, G, L, Dq), device=dev, dtype=torch.uint8)
            v = torch.randint(0, 255, (Bd, G, L, Dq), device=dev, dtype=torch.uint8)
            s = torch.rand(Bd, G, L, device=dev) * 0.01
            z = torch.randint(0, 15, (Bd, G, L), device=dev, dtype=torch.int32)
            for _ in range(args.iters):
                cu.decode_attention(q, k, v, scale, L, True, quant=(s, z, s, z, args.bits))
    elif args.which == "allreduce":
        # one rank: the kernel runs its barrier, pull, reduce and push paths on local memory only
        import os

        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        from keys_values_b200.parallel.symm import SymmetricArena

        n = 128 * 2**20
        arena = SymmetricArena(n, torch.bfloat16, dev, 1, 0)
        arena.tensor.normal_()
        for _ in range(args.iters):
            arena.all_reduce_mean_(0, n)
        torch.cuda.synchronize()
        arena.close()
        dist.destroy_process_group()
    else:
        raise SystemExit(f"unknown case {args.which}")
    torch.cuda.synchronize()
    cu.check_status(dev)
    print("done")


if __name__ == "__main__":
    main()
