"""Worker for the multi-GPU tests: launched once per rank by ``test_multi_gpu.py``.

Usage: python dist_worker.py <case> <rank> <world> <port> [backend]
Every case compares the framework's own collective / data-parallel path with the
single-process result or with NCCL, and prints ``OK`` on success.
"""
import os
import sys
import zlib
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
        # identical bits on every rank after a full reduction
        arena.tensor.copy_(torch.randn(n, device=dev, dtype=torch.float32, generator=g).to(dtype))
        arena.all_reduce_mean_(0, n)
        torch.cuda.synchronize(dev)
        mine = arena.tensor.clone()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        for other in gathered:
            assert torch.equal(other, mine)
        arena.close()


def case_dp_train_full(rank, world, dev):
    """Data-parallel step with every parameter trainable (embeddings, head and norms too): their
    arena slots are not neighbours, and the embedding gradient is accumulated last."""
    case_dp_train(rank, world, dev, train_all_parameters=True)


def case_dp_train(rank, world, dev, train_all_parameters=False):
    """Data-parallel LoRA step: gradients after the reducer equal the mean of the per-rank
    gradients computed without it."""
    from keys_values_b200.finetune.engine import build_lora_training_setup

    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    kw = dict(cache_name="h2o-torch-quantized8", cache_length=128, chunk_size=32, lora_r=4, lora_alpha=8, micro_batch_size=1,
              yarn_rope=False, seed=7, train_all_parameters=train_all_parameters)
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
    if train_all_parameters:
        assert "transformer.wte.weight" in ref and "lm_head.weight" in ref or "lm_head.linear.weight" in ref
    for n, p in setup.gpt_model.named_parameters():
        if n in ref:
            tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
            torch.testing.assert_close(p.grad.float(), ref[n], atol=tol, rtol=tol, msg=lambda m: f"{n}: {m}")


def case_tp_ops(rank, world, dev):
    """Fused all-gather→GEMM and GEMM→reduce-scatter against NCCL + a library matmul."""
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.parallel.tp import TPContext

    rows, K, N = 256, 512, 768
    ctx = TPContext(world, rank, dev, max_rows=world * rows, max_features=1024, copy_ctas=4)
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    for it in range(3):
        # all-gather → GEMM
        shard = torch.randn(rows, K, device=dev, dtype=torch.bfloat16, generator=g)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
        ctx.stage_view(rows, K).copy_(shard)
        out = ctx.allgather_gemm(rows, w)
        full = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(full, shard)
        ref = torch.cat(full).float() @ w.float().t()
        torch.cuda.synchronize(dev)
        cu.check_status(dev)
        torch.testing.assert_close(out.float(), ref, atol=0.15, rtol=3e-2)
        # GEMM → reduce-scatter (+ residual)
        M = world * rows
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, generator=g)
        w2 = torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
        res = torch.randn(rows, N, device=dev, dtype=torch.bfloat16, generator=g)
        out2 = ctx.gemm_reduce_scatter(x, w2, residual=res)
        part = (x.float() @ w2.float().t()).to(torch.bfloat16).float()
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        ref2 = part[rank * rows : (rank + 1) * rows] + res.float()
        torch.cuda.synchronize(dev)
        cu.check_status(dev)
        torch.testing.assert_close(out2.float(), ref2, atol=0.25, rtol=3e-2)
    ctx.close()


def case_tp_model(rank, world, dev):
    """Tensor-parallel chunked forward with H2O caches equals the single-GPU forward."""
    import dataclasses

    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.models.model import GPT
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.parallel.tp import TPContext, TPModel

    torch.manual_seed(3)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        gpt = GPT.from_name("tiny-qwen3")
    torch.set_default_dtype(prev)
    gpt.apply(gpt._init_weights)
    cfg = gpt.config
    T0, Tc, C = 256, 256, 512
    ids = torch.randint(0, cfg.vocab_size, (1, T0 + 2 * Tc), device=dev)
    dist.broadcast(ids, 0)
    name = "lastrec-default"
    # single GPU reference
    gpt.assign_kv_caches(KVCacheFactory.create(gpt, name, 1, C, dtype=torch.bfloat16, device=dev))
    gpt.max_seq_length = ids.shape[1]
    with torch.no_grad():
        gpt.reset()
        refs = [gpt(ids[:, :T0], skip_lm_head=True)]
        for s in range(T0, ids.shape[1], Tc):
            refs.append(gpt(ids[:, s : s + Tc], skip_lm_head=True))
    # tensor parallel
    ctx = TPContext(world, rank, dev, max_rows=256, max_features=max(cfg.n_embd, cfg.intermediate_size), copy_ctas=4)

    def make_cache(block_idx, g_local, h_local):
        lc = dataclasses.replace(cfg, n_head=h_local, n_query_groups=g_local)
        return KVCacheFactory.create_single(name, lc, 1, C, block_idx, device=dev, dtype=torch.bfloat16, cache_kwargs=dict(mha=gpt.mha))

    tpm = TPModel(gpt, ctx, make_cache)
    tpm.reset()
    pos = 0
    for ref_chunk, n in zip(refs, [T0, Tc, Tc]):
        chunk_ids = ids[:, pos : pos + n]
        x = gpt.embed(chunk_ids)[0]
        rows = n // world
        out = tpm.forward_hidden(x[rank * rows : (rank + 1) * rows].contiguous(), chunk_ids)
        torch.cuda.synchronize(dev)
        cu.check_status(dev)
        want = ref_chunk[0, rank * rows : (rank + 1) * rows].float()
        err = (out.float() - want).norm() / want.norm()
        assert err < 5e-2, f"chunk at {pos}: relative error {err}"
        pos += n
    ctx.close()


def case_tp_gpt(rank, world, dev):
    """The sharded model through the ordinary stack (prefill, chunks, single-token decode steps, batch 2, H2O
    caches that evict) equals the whole model; on GPUs the decode steps also run as a captured graph."""
    from keys_values_b200.config import Config
    from keys_values_b200.generate.decode_graph import Decoder
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.models.model import GPT
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.parallel.tp import TPComm, TPGPT, shard_state_dict

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(5)
    cfg = Config.from_name(os.environ.get("KVB200_TEST_MODEL", "tiny-qwen3"))
    full = GPT(cfg)
    full.apply(full._init_weights)
    full = full.to(device=dev, dtype=dtype).eval()
    comm = TPComm(world, rank, dev, dtype=dtype)
    shard = TPGPT(cfg, comm).to(device=dev, dtype=dtype).eval()
    shard.load_state_dict(shard_state_dict(full.state_dict(), cfg, world, rank))
    B, T0, Tc, C, n_dec = 2, 192, 64, 256, 6
    ids = torch.randint(0, cfg.vocab_size, (B, T0 + 3 * Tc + n_dec), device=dev)
    dist.broadcast(ids, 0)
    name = "h2o-default"
    outs = []
    for model in (full, shard):
        model.assign_kv_caches(KVCacheFactory.create(model, name, B, C, dtype=dtype, device=dev, cache_kwargs=dict(max_chunk_size=Tc)))
        model.max_seq_length = ids.shape[1]
        model.reset()
        res = []
        with torch.no_grad():
            res.append(model(ids[:, :T0])[:, -1])
            pos = T0
            for _ in range(3):
                res.append(model(ids[:, pos : pos + Tc])[:, -1])
                pos += Tc
            decoder = Decoder(model, B, use_graph=cuda, warmup=2)
            for _ in range(n_dec):
                res.append(decoder(ids[:, pos : pos + 1])[:, -1].clone())
                pos += 1
            if cuda:
                assert decoder.graph is not None, decoder.reason
        outs.append(torch.stack(res).float())
    if cuda:
        torch.cuda.synchronize(dev)
        cu.check_status(dev)
    want, got = outs
    err = (got - want).norm() / want.norm()
    assert err < (3e-2 if cuda else 1e-4), f"relative error of the logits {err}"
    # every rank holds the same bits (the sum runs in rank order everywhere)
    gathered = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(gathered, got)
    if cuda:
        assert all(torch.equal(g, got) for g in gathered)
    comm.close()


def case_tp_gpt_grads(rank, world, dev):
    """Training through the sharded model: the gradients of a rank's shard are the matching slices of the
    whole model's gradients, those of replicated parameters (norms, embedding, head) are equal on every rank."""
    from keys_values_b200.config import Config
    from keys_values_b200.models.model import GPT
    from keys_values_b200.parallel.tp import TPComm, TPGPT, shard_state_dict

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(6)
    cfg = Config.from_name("tiny-qwen3")
    full = GPT(cfg)
    full.apply(full._init_weights)
    full = full.to(device=dev, dtype=dtype)
    comm = TPComm(world, rank, dev, dtype=dtype)
    shard = TPGPT(cfg, comm).to(device=dev, dtype=dtype)
    shard.load_state_dict(shard_state_dict(full.state_dict(), cfg, world, rank))
    ids = torch.randint(0, cfg.vocab_size, (2, 96), device=dev)
    tg = torch.randint(0, cfg.vocab_size, (2 * 96,), device=dev)
    dist.broadcast(ids, 0)
    dist.broadcast(tg, 0)
    losses = []
    for model in (full, shard):
        logits = model(ids)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), tg)
        loss.backward()
        losses.append(loss.detach().float())
    assert abs(losses[0] - losses[1]) < (2e-2 if cuda else 1e-5), losses
    want = shard_state_dict({n: p.grad for n, p in full.named_parameters()}, cfg, world, rank)
    tol = 6e-2 if cuda else 1e-4
    for n, p in shard.named_parameters():
        assert p.grad is not None, n
        w, g = want[n].float(), p.grad.float()
        err = (g - w).norm() / w.norm().clamp(min=1e-6)
        assert err < tol, f"{n}: relative gradient error {err}"
    comm.close()


def case_tp_lora_grads(rank, world, dev):
    """LoRA under tensor parallelism (A of column-parallel and B of row-parallel linears replicated, the other
    factor sharded): loss and the gradients of all adapter tensors equal those of the whole LoRA model."""
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.parallel.tp import TPComm, TPLoRAGPT, shard_state_dict

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(8)
    cfg = lora_mod.Config.from_name("tiny-qwen3", lora_r=4, lora_alpha=8, lora_query=True, lora_key=True, lora_value=True,
                                    lora_projection=True, lora_mlp=True)
    full = lora_mod.GPT(cfg)
    full.apply(full._init_weights)
    for n, p in full.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(full)
    full = full.to(device=dev, dtype=dtype)
    comm = TPComm(world, rank, dev, dtype=dtype)
    shard = TPLoRAGPT(cfg, comm).to(device=dev, dtype=dtype)
    shard.load_state_dict(shard_state_dict(full.state_dict(), cfg, world, rank))
    lora_mod.mark_only_lora_as_trainable(shard)
    ids = torch.randint(0, cfg.vocab_size, (2, 80), device=dev)
    tg = torch.randint(0, cfg.vocab_size, (2 * 80,), device=dev)
    dist.broadcast(ids, 0)
    dist.broadcast(tg, 0)
    losses = []
    for model in (full, shard):
        logits = model(ids)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), tg)
        loss.backward()
        losses.append(loss.detach().float())
    assert abs(losses[0] - losses[1]) < (2e-2 if cuda else 1e-5), losses
    want = shard_state_dict({n: p.grad for n, p in full.named_parameters() if p.grad is not None}, cfg, world, rank)
    tol = 8e-2 if cuda else 1e-4
    n_checked = 0
    for n, p in shard.named_parameters():
        if not p.requires_grad:
            continue
        w, g = want[n].float(), p.grad.float()
        err = (g - w).norm() / w.norm().clamp(min=1e-6)
        assert err < tol, f"{n}: relative gradient error {err}"
        n_checked += 1
    assert n_checked >= 2 * 10  # A and B of qkv, proj, fc_1, fc_2, mlp.proj in both layers
    # a checkpoint written under tensor parallelism is the whole model's
    from keys_values_b200.parallel.tp import gather_whole_state_dict

    whole = gather_whole_state_dict(shard, only_trainable=True)
    if rank == 0:
        ref_sd = {k: v.cpu() for k, v in full.state_dict().items() if "lora_" in k}
        assert set(whole) == set(ref_sd)
        for k, v in ref_sd.items():
            assert torch.equal(whole[k], v), k
    else:
        assert whole is None
    comm.close()


def case_tp_train(rank, world, dev):
    """The chunked gradient engine (cells, activation checkpoints, replay through the cache) on a LoRA shard:
    loss and adapter gradients equal the whole model's; every rank evicts for its own KV heads."""
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.models.head_model import CrossEntropyOnLogits
    from keys_values_b200.parallel.tp import TPComm, TPLoRAGPT, shard_state_dict

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(9)
    cfg = lora_mod.Config.from_name("tiny-qwen3", lora_r=4, lora_alpha=8, lora_query=True, lora_value=True, lora_projection=True)
    full = lora_mod.GPT(cfg)
    full.apply(full._init_weights)
    for n, p in full.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(full)
    full = full.to(device=dev, dtype=dtype)
    comm = TPComm(world, rank, dev, dtype=dtype)
    shard = TPLoRAGPT(cfg, comm).to(device=dev, dtype=dtype)
    shard.load_state_dict(shard_state_dict(full.state_dict(), cfg, world, rank))
    lora_mod.mark_only_lora_as_trainable(shard)
    T, C, cs = (1024, 256, 128) if cuda else (320, 96, 32)
    ids = torch.randint(0, cfg.vocab_size, (1, T), device=dev)
    tg = torch.randint(0, cfg.vocab_size, (1, cs), device=dev)
    dist.broadcast(ids, 0)
    dist.broadcast(tg, 0)
    for name, exact in (("lastrec-default", True), ("h2o-torch-quantized8", False)):
        losses, grads = [], []
        for model in (full, shard):
            for p in model.parameters():
                p.grad = None
            ck = dict(max_chunk_size=cs) if "h2o" in name else None
            model.assign_kv_caches(KVCacheFactory.create(model, name, 1, C, dtype=dtype, device=dev, cache_kwargs=ck))
            gm = LongContextGradientModel(model, CrossEntropyOnLogits(model.config), layers_per_cell=1, chunk_size=cs)
            gm.train()
            loss = gm(ids, tg)
            loss.backward()
            losses.append(float(loss))
            grads.append({n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None})
        tol = (3e-2 if cuda else 1e-4) if exact else 5e-2
        assert abs(losses[0] - losses[1]) < tol * max(1.0, abs(losses[0])), (name, losses)
        if exact:
            want = shard_state_dict(grads[0], cfg, world, rank)
            for n, g in grads[1].items():
                w = want[n].float()
                err = (g.float() - w).norm() / w.norm().clamp(min=1e-6)
                assert err < (8e-2 if cuda else 1e-3), f"{name} {n}: relative gradient error {err}"
    if cuda:
        from keys_values_b200.ops import cuda as cu

        torch.cuda.synchronize(dev)
        cu.check_status(dev)
    comm.close()


def case_dp_tp_train(rank, world, dev):
    """Data parallel x tensor parallel (world 4 = 2 replicas x 2 shards): after the step's reductions every rank
    holds its shard of the MEAN over the replicas of the whole model's gradients; one optimizer step with
    clipping keeps replicated parameters equal on all ranks."""
    from keys_values_b200.finetune.engine import build_lora_training_setup, training_step
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.models.head_model import CrossEntropyOnLogits
    from keys_values_b200.models.pos_encoding import position_encoding_factory
    from keys_values_b200.parallel.tp import shard_state_dict, unshard_state_dict

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    tp = 2
    dp_rank, tp_rank = rank // tp, rank % tp
    T, C, cs = (512, 128, 64) if cuda else (192, 64, 32)
    setup = build_lora_training_setup("tiny-qwen3", dev, dtype, cache_name="lastrec-default", cache_length=C, chunk_size=cs, lora_r=4,
                                      lora_alpha=8, micro_batch_size=1, world_size=world, rank=rank, yarn_rope=False, seed=11,
                                      max_norm=0.5, tp_size=tp, overlap_allreduce=cuda)
    cfg = setup.config
    with torch.no_grad():
        for n, p in setup.gpt_model.named_parameters():
            if "lora_B" in n:  # same values on every rank: seeded by name
                g = torch.Generator().manual_seed(zlib.crc32(n.encode()) % 10_000)
                p.copy_((torch.randn(p.shape, generator=g) * 0.05).to(p))
    # the whole model, rebuilt on every rank from the shards of replica 0
    shards = [None] * world
    dist.all_gather_object(shards, {k: v.detach().cpu() for k, v in setup.gpt_model.state_dict().items()})
    whole_sd = unshard_state_dict(shards[:tp], cfg)
    whole = lora_mod.GPT(cfg, pos_encoding=position_encoding_factory(cfg, do_yarn=False, device=dev))
    whole.load_state_dict(whole_sd)
    whole = whole.to(device=dev, dtype=dtype)
    lora_mod.mark_only_lora_as_trainable(whole)
    gen = torch.Generator().manual_seed(21)
    data = [(torch.randint(0, cfg.vocab_size, (1, T), generator=gen), torch.randint(0, cfg.vocab_size, (1, cs), generator=gen)) for _ in range(world // tp)]
    mean_grads = None
    for ids, tg in data:
        for p in whole.parameters():
            p.grad = None
        whole.assign_kv_caches(KVCacheFactory.create(whole, "lastrec-default", 1, C, dtype=dtype, device=dev))
        gm = LongContextGradientModel(whole, CrossEntropyOnLogits(cfg), layers_per_cell=1, chunk_size=cs)
        gm.train()
        gm(ids.to(dev), tg.to(dev)).backward()
        gr = {n: p.grad.detach().float() / len(data) for n, p in whole.named_parameters() if p.grad is not None}
        mean_grads = gr if mean_grads is None else {n: mean_grads[n] + g for n, g in gr.items()}
    want = shard_state_dict(mean_grads, cfg, tp, tp_rank)
    # this rank's step on the batch of its replica, without the optimizer: forward, backward, reductions
    ids, tg = data[dp_rank]
    setup.optimizer.zero_grad(set_to_none=False)
    setup.grad_reducer.begin_step()
    setup.model(ids.to(dev), tg.to(dev)).backward()
    setup.grad_reducer.finish_step()
    if cuda:
        torch.cuda.synchronize(dev)
    for n, p in setup.gpt_model.named_parameters():
        if p.requires_grad:
            w = want[n].to(dev)
            err = (p.grad.float() - w).norm() / w.norm().clamp(min=1e-6)
            assert err < (0.1 if cuda else 1e-3), f"{n}: relative gradient error {err}"
    # a full step (with clipping by the whole model's norm): replicated tensors stay equal everywhere
    loss = training_step(setup, ids.to(dev), tg.to(dev))
    assert torch.isfinite(loss)
    rep = torch.cat([p.detach().float().reshape(-1) for n, p in setup.gpt_model.named_parameters() if n.endswith("attn.qkv.lora_A")])
    everyone = [torch.empty_like(rep) for _ in range(world)]
    dist.all_gather(everyone, rep)
    for other in everyone:
        torch.testing.assert_close(other, rep, atol=0 if not cuda else 1e-6, rtol=0)
    setup.extras["tp_comm"].close()


def case_tp_vocab_ce(rank, world, dev):
    """Vocabulary-parallel cross-entropy: per-row losses, and the gradients with respect to the hidden states and the
    head's weight, equal those of the whole-vocabulary loss (ignored targets included; vocabulary not divisible by the
    number of ranks); the fused all-reduce + residual + RMSNorm falls back to separate ops off the GPU."""
    from keys_values_b200.parallel.tp import TPComm, vocab_parallel_cross_entropy

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    comm = TPComm(world, rank, dev, dtype=dtype)
    g = torch.Generator().manual_seed(4)
    rows, E, V = 37, 64, 1001
    x0 = torch.randn(rows, E, generator=g).to(dev, dtype)
    w0 = (torch.randn(V, E, generator=g) * 0.2).to(dev, dtype)
    tg = torch.randint(0, V, (rows,), generator=g).to(dev)
    tg[::5] = -100
    x1, w1 = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    want = torch.nn.functional.cross_entropy((x1 @ w1.t()).float(), tg, ignore_index=-100, reduction="none")
    want.sum().backward()
    x2, w2 = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    got = vocab_parallel_cross_entropy(x2, w2, tg, comm)
    got.sum().backward()
    tol = dict(atol=3e-2, rtol=3e-2) if cuda else dict(atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(got, want, **tol)
    torch.testing.assert_close(x2.grad.float(), x1.grad.float(), **tol)
    torch.testing.assert_close(w2.grad.float(), w1.grad.float(), **tol)
    # all-reduce + residual + RMSNorm in one call
    part = torch.randn(4, E, generator=g).to(dev, dtype) + rank
    res = torch.randn(4, E, generator=g).to(dev, dtype)
    nw = torch.rand(E, generator=g).to(dev, dtype)
    buf = comm.out_buffer(4, E, dtype)
    buf.copy_(part)
    x, normed = comm.all_reduce_add_norm(buf, res, nw, 1e-5)
    total = part.float().clone()
    dist.all_reduce(total)
    want_x = (total + res.float()).to(dtype)
    wf = want_x.float()
    want_n = (wf * torch.rsqrt(wf.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()).to(dtype)
    torch.testing.assert_close(x.float(), want_x.float(), **tol)
    torch.testing.assert_close(normed.float(), want_n.float(), **tol)
    comm.close()


if __name__ == "__main__":
    main()
