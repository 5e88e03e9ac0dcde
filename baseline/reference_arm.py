"""Reference arm of ``bench.py``: the unmodified reference library from ``baseline/_ref``.

What runs here is the reference's own training path, built through its own functions
in the order its ``finetune_long_lora`` command uses them
(``keys_values/finetune/longcontext_full.py:main``): ``get_mha_and_cache_kwargs`` →
``create_gpt_model`` (LoRA ``GPT``) → ``HeadModelFactory.create`` → ``wrap_gpt_model``
(``KVCacheFactory.create`` + ``LongContextGradientModel``) → ``instantiate_torch_optimizer``,
and then the body of its ``fit`` loop (``:1493-1650``): ``loss = model(input_ids, targets)``,
``loss.backward()``, ``CPUOffloadAccumulateGradients`` all-reduce (NCCL) of the flat gradients,
loss all-reduce, gradient clipping, ``optimizer.step()``, ``gc.collect()`` and
``torch.cuda.empty_cache()``. Arguments are the defaults of that command except where the
benchmark config names a value (LoRA on q/k/v/o, micro-batch 1, cache / chunk sizes).

Nothing of this repository's models, kernels or engine is imported on this path. The
packages the reference imports but that are not installed (LitGPT, Lightning, torchmetrics,
jsonargparse) are replaced by the plain-PyTorch stand-ins under ``baseline/shim``. The
reference's CUDA extension is its own source compiled with an added sm_100 target
(``baseline/install_reference.py``); which attention path was active is reported in the
``attention_path`` field of the result.
"""
from __future__ import annotations

import gc
import importlib
import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE / "_ref"
SHIM_ROOT = HERE / "shim"


# Small architectures for CPU checks of this arm (not benchmark configs).
TINY_CONFIGS = {
    "tiny-qwen3": dict(
        name="tiny-qwen3", block_size=4096, vocab_size=512, padded_vocab_size=512, n_layer=2, n_head=4, n_embd=64,
        n_query_groups=2, head_size=16, rotary_percentage=1.0, parallel_residual=False, bias=False,
        norm_class_name="RMSNorm", mlp_class_name="LLaMAMLP", intermediate_size=172, norm_eps=1e-6, rope_base=10000,
        norm_qk=True,
    ),
}


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why[:400]}


def _import_reference():
    if not (REF_ROOT / "keys_values").is_dir():
        raise ImportError("baseline/_ref is missing (run the offline pip install of the reference with --target baseline/_ref)")
    for p in (str(SHIM_ROOT), str(REF_ROOT)):
        if p not in sys.path:
            sys.path.insert(0, p)
    return importlib.import_module("keys_values.finetune.longcontext_full")


def _attention_path(lcf, sdpa_args) -> str:
    """Says which of the reference's SDPA-with-weights paths is active in this process."""
    try:
        if sdpa_args.flashinfer_attention and lcf.get_flashinfer_sdpa() is not None:
            return "reference FlashInfer extension (own sources, sm_100 build) + Triton score-sum; FlexAttention elsewhere"
    except Exception:
        pass
    if sdpa_args.flex_attention and sdpa_args.use_flex_for_attn_weights:
        return "2x FlexAttention (the reference's extension is not loadable)"
    return "eager blockwise SDPA"


def run_reference(args) -> dict:
    try:
        lcf = _import_reference()
    except Exception as ex:
        return _unavailable(f"import of the reference failed: {type(ex).__name__}: {ex}")
    import torch
    import torch.distributed as dist

    on_cpu = not torch.cuda.is_available()
    if on_cpu and not getattr(args, "ref_allow_cpu", False):
        return _unavailable("the reference's fine-tuning path needs a CUDA device")

    import lightning as L  # the stand-in
    from keys_values.finetune.args import GradientArgs, KVCacheArgs, OptimizerArgs, SDPAArgs
    from keys_values.head_model import CrossEntropyOnLogits
    from keys_values.head_model_factory import HeadModelFactory
    from keys_values.lora import Config as ConfigLoRA
    from keys_values.optimize.grad_accumulate import CPUOffloadAccumulateGradients
    from keys_values.utils import VerbosityLevels
    from litgpt.config import name_to_config
    from litgpt.utils import instantiate_torch_optimizer

    from bench import ClockSampler  # clock sampling only; no model or kernel code

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    fabric = L.Fabric(devices=world, precision="32-true" if on_cpu else "bf16-true")
    fabric.launch()
    dev = fabric.device
    if not on_cpu:
        torch.cuda.set_device(dev)
    fabric.seed_everything(1337 + rank)

    conf = dict(name_to_config[args.model]) if args.model in name_to_config else dict(TINY_CONFIGS[args.model])
    if args.n_layer is not None:
        conf["n_layer"] = args.n_layer
    config = ConfigLoRA(**conf, lora_r=8, lora_alpha=16, lora_dropout=0.0, lora_query=True, lora_key=True,
                        lora_value=True, lora_projection=True, lora_mlp=False, lora_head=False, lora_kind="default")
    kv_cache = KVCacheArgs(
        name=args.cache_name, cache_length=args.cache_length, chunk_size=args.chunk_size,
        cache_kwargs={"replay_log_blocksize": 1024, "max_num_ranges": 4},
        randomize_chunk_sizes=False, allocate_buffers=False,
    )
    grad = GradientArgs(layers_per_cell=1, chunks_per_cell_multiplier=1.0, layercp_qname=None, cachecp_qname=None,
                        single_tokens_for_targets=False, max_match_trials_pack_arg=8,
                        layercp_pin_memory=not on_cpu, cachecp_pin_memory=not on_cpu)
    # FlexAttention has no backward on the CPU: the CPU debug run uses the reference's zero-padded SDPA path.
    sdpa = SDPAArgs(flex_attention=not on_cpu, flex_extend_kv=False, flex_num_q_lens=4)
    from keys_values.attention import flashinfer_ops as ref_ext

    if not ref_ext.is_available():
        # Without its extension the reference's own fallback for the summed weights is 2x FlexAttention.
        sdpa.flashinfer_attention = False
    if getattr(args, "ref_fused", False):
        sdpa.fused_rope = sdpa.fused_rmsnorm = sdpa.fused_swiglu = True
    lcf.set_fused_rope_enabled(sdpa.fused_rope)
    lcf.set_fused_rmsnorm_enabled(sdpa.fused_rmsnorm)
    lcf.set_fused_swiglu_enabled(sdpa.fused_swiglu)

    dtype = torch.float32 if on_cpu else torch.bfloat16
    with fabric.init_module(empty_init=(world > 1)):
        kv_cache = kv_cache.update_cache_kwargs()
        mha_kwargs = lcf.get_mha_and_cache_kwargs(4, config, kv_cache, sdpa, True, fabric, world)
        torch.set_default_dtype(dtype)
        gpt_model = lcf.create_gpt_model(config, **mha_kwargs)
        head_model = HeadModelFactory.create(name=CrossEntropyOnLogits.NAME, config=config, data=None)
        lcf.adapt_requires_grad(gpt_model, head_model)
        model, _ = lcf.wrap_gpt_model(
            gpt_model=gpt_model, head_model=head_model, kv_cache=kv_cache, grad=grad, verbose=VerbosityLevels.NONE,
            attention_backward_temp_size_gb=2, max_batch_size=1, dtype=dtype, average_loss_per_batch=True,
            fabric=fabric,
        )
    torch.set_default_dtype(torch.float32)
    opt_args = OptimizerArgs(name="AdamW")
    optimizer = instantiate_torch_optimizer(opt_args.name, model.parameters(), **opt_args.optimizer_kwargs())
    grad_reducer = CPUOffloadAccumulateGradients(group=list(range(world)), fabric=fabric)
    attention_path = _attention_path(lcf, sdpa)

    vocab = config.vocab_size
    gen = torch.Generator().manual_seed(99 + rank)

    def new_batch():
        ids = torch.randint(0, vocab, (1, args.seq_len), generator=gen)
        tg = torch.randint(0, vocab, (1, args.num_targets), generator=gen)
        return (ids, tg) if on_cpu else (ids.pin_memory(), tg.pin_memory())

    h2d_bytes = 8 * (args.seq_len + args.num_targets)

    def step(ids_host, tg_host):
        """The body of the reference's ``fit`` loop for one batch; returns the loss as a Python float."""
        ids = ids_host.to(dev, non_blocking=True)
        tg = tg_host.to(dev, non_blocking=True)
        loss = model(input_ids=ids, targets=tg, scale_factor=1.0)
        loss.backward()
        module_pairs = [(model.gpt_model, None)]
        if model.head_model.parameters():
            module_pairs.append((model.head_model, None))
        grad_reducer(module_pairs=module_pairs, mean_reduction=True)
        fabric.all_reduce(loss, reduce_op="mean")
        value = float(loss.detach().float().cpu())  # running_loss.update(...) + logging read it every step
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        del loss
        gc.collect()
        if not on_cpu:
            torch.cuda.empty_cache()
        return value

    def sync():
        if world > 1:
            dist.barrier()
        if not on_cpu:
            torch.cuda.synchronize(dev)

    # ---- warm-up (the first step also compiles the FlexAttention graphs)
    budget_s = float(getattr(args, "ref_time_budget", 1500.0))
    t_start = time.perf_counter()
    warmup, steps = args.warmup, args.steps
    step_s = None
    done_warm = 0
    while done_warm < warmup:
        t0 = time.perf_counter()
        step(*new_batch())
        sync()
        step_s = time.perf_counter() - t0
        done_warm += 1
        if done_warm >= 2:
            # Fit the run into the time budget: keep three warm-up steps in total if they were asked for,
            # give the rest of the budget to timed steps (at least one).
            left = budget_s - (time.perf_counter() - t_start)
            t = torch.tensor([left / max(step_s, 1e-3)], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
            can_do = int(t.item())
            if can_do < (warmup - done_warm) + steps:
                more_warm = max(0, min(warmup, 3) - done_warm)
                steps = max(1, min(steps, can_do - more_warm))
                warmup = done_warm + more_warm
    batches = [new_batch() for _ in range(steps)]
    sync()
    sampler = None if on_cpu else ClockSampler(dev.index or 0)
    if sampler is not None:
        sampler.start()
    dev_ms = 0.0
    losses = []
    t0 = time.perf_counter()
    for ids, tg in batches:
        if on_cpu:
            t1 = time.perf_counter()
            losses.append(step(ids, tg))
            dev_ms += (time.perf_counter() - t1) * 1e3
            continue
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        losses.append(step(ids, tg))
        e1.record()
        e1.synchronize()
        dev_ms += e0.elapsed_time(e1)
    sync()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if sampler is not None else None
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    tokens = args.seq_len * world * steps
    reduced = args.n_layer is not None or args.seq_len != 131072 or args.model != "Qwen3-4B"
    result = {
        "metric": "long-ctx LoRA train tokens/s/box",
        "value": tokens / (dev_ms / 1e3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "steps_requested": args.steps,
        "warmup_requested": args.warmup,
        "ms_per_step": dev_ms / steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp32 (CPU debug run)" if on_cpu else "bf16",
        "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "reference",
        "attention_path": attention_path,
        "config": {
            "model": f"{args.model}-architecture" + (f" (REDUCED to {args.n_layer} layers)" if args.n_layer else ""),
            "global_batch": world, "seq_len": args.seq_len, "parallelism": f"dp{world}",
            "lora": "r=8 alpha=16 on q,k,v,o", "cache": args.cache_name, "cache_length": args.cache_length,
            "chunk_size": args.chunk_size, "loss_tokens": args.num_targets, "optimizer": "AdamW",
            "l2": "per-step working set exceeds the 126 MB L2",
            "note": ("value sums CUDA-event times around each step; e2e is the wall clock of the same steps "
                     "(the reference's loop copies the batch to the device and reads the loss every step); "
                     "steps/warmup are lowered from the requested numbers when the run would not fit the time budget"),
        },
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / steps},
        "gpu_launches": None,
        "loss": losses[-1] if losses else None,
        "peak_mem_gb": None if on_cpu else torch.cuda.max_memory_allocated(dev) / 2**30,
        "reduced": reduced,
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_reference_inference(args) -> dict:
    """Config 4 through the reference's own generation path on ONE GPU (it has no tensor parallelism): the
    construction sequence of its ``generate`` command (``keys_values/generate/base.py:436-640``: ``GPT(config)`` →
    ``KVCacheFactory.create`` → ``LongContextInferenceModel`` → ``batched_generate_fn``) with random-init weights of
    the named architecture. The first yield of its generator is the chunked prompt pass plus one sample (prefill),
    the remaining yields are its single-token steps (decode); both are timed with CUDA events."""
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return _unavailable("the reference has no tensor parallelism: its inference arm runs on one GPU only")
    try:
        _import_reference()
    except Exception as ex:
        return _unavailable(f"import of the reference failed: {type(ex).__name__}: {ex}")
    import torch

    on_cpu = not torch.cuda.is_available()
    if on_cpu and not getattr(args, "ref_allow_cpu", False):
        return _unavailable("the reference's inference arm is timed on a CUDA device")
    from keys_values.config import Config
    from keys_values.generate.base import batched_generate_fn
    from keys_values.kvcache.factory import KVCacheFactory
    from keys_values.long_context import LongContextInferenceModel
    from keys_values.model import GPT
    from litgpt.config import name_to_config

    from bench import ClockSampler  # clock sampling only; no model or kernel code

    model_name = "Llama-3-8B" if args.model == "Qwen3-4B" else args.model
    seq = 65536 if args.seq_len == 131072 else args.seq_len
    cache_name = "h2o-torch-quantized4" if args.cache_name == "h2o-torch-quantized8" else args.cache_name
    cache_length = 8192 if args.cache_length == 16384 else args.cache_length
    chunk = 2048 if args.chunk_size == 1024 else args.chunk_size
    conf = dict(name_to_config[model_name]) if model_name in name_to_config else dict(TINY_CONFIGS[model_name])
    if args.n_layer is not None:
        conf["n_layer"] = args.n_layer
    config = Config(**conf)
    dev = torch.device("cpu") if on_cpu else torch.device("cuda", 0)
    dtype = torch.float32 if on_cpu else torch.bfloat16
    torch.manual_seed(0)
    torch.set_default_dtype(dtype)
    try:
        with torch.device(dev):
            gpt_model = GPT(config)
    finally:
        torch.set_default_dtype(torch.float32)
    gpt_model.apply(gpt_model._init_weights)
    gpt_model.assign_kv_caches(KVCacheFactory.create(gpt_model=gpt_model, name=cache_name, max_batch_size=args.batch, cache_length=cache_length,
                                                     device=dev, dtype=dtype, cache_kwargs={"max_chunk_size": chunk} if "h2o" in cache_name else None))
    gpt_model.eval()
    model = LongContextInferenceModel(gpt_model=gpt_model, head_model=None, chunk_size=chunk)
    gen = torch.Generator().manual_seed(7)
    host_prompts = torch.randint(0, config.vocab_size, (args.batch, seq), generator=gen)
    if not on_cpu:
        host_prompts = host_prompts.pin_memory()
    greedy = dict(temperature=0.0, top_p=0.0)
    sampler = ClockSampler(0)
    if not on_cpu:
        sampler.start()

    def event():
        if on_cpu:
            return time.perf_counter()
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def elapsed(a, b):
        return (b - a) if on_cpu else a.elapsed_time(b) / 1e3

    with torch.inference_mode():
        # warm-up on a short prompt: kernel loading, Triton compilation, allocator
        short = host_prompts[:, : min(seq, 2 * cache_length)].to(dev)
        for k, _ in enumerate(batched_generate_fn(model, short, 4, sample_args=greedy)):
            pass
        if not on_cpu:
            torch.cuda.synchronize(dev)
        e0 = event()
        prompts = host_prompts.to(dev, non_blocking=True)
        out, e1 = [], None
        for tokens in batched_generate_fn(model, prompts, args.decode, sample_args=greedy):
            out.append(tokens)
            if e1 is None:
                e1 = event()  # the prompt pass and the first sampled token are behind us
        host_tokens = torch.cat(out, dim=1).cpu()
        e2 = event()
        if not on_cpu:
            torch.cuda.synchronize(dev)
    t_pre, t_dec = elapsed(e0, e1), elapsed(e1, e2)
    n_dec = max(host_tokens.shape[1] - 1, 1)
    clocks = sampler.stop() if not on_cpu else {}
    total = args.batch * (seq + host_tokens.shape[1]) / (t_pre + t_dec)
    return {
        "metric": "long-ctx inference tokens/s (prefill + decode)", "value": total, "unit": "tokens/s", "n_gpus": 1, "steps": 1,
        "warmup": args.warmup, "ms_per_step": 1e3 * (t_pre + t_dec), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32" if on_cpu else "bf16", "data": "synthetic uniform-random token ids, random-init weights", "impl": "reference",
        "prefill_tokens_per_s": args.batch * seq / t_pre, "decode_tokens_per_s": args.batch * n_dec / t_dec,
        "ms_per_decode_step": 1e3 * t_dec / n_dec,
        "config": {"model": model_name + "-architecture" + (f" (REDUCED to {args.n_layer} layers)" if args.n_layer else ""),
                   "global_batch": args.batch, "seq_len": seq, "parallelism": "tp1", "cache": cache_name, "cache_length": cache_length,
                   "chunk_size": chunk, "decode_tokens": int(host_tokens.shape[1]),
                   "note": "the reference's generate path: chunked prompt pass, then eager single-token steps"},
        "clocks": clocks,
        "e2e": {"value": total, "unit": "tokens/s", "h2d_bytes_per_step": host_prompts.numel() * host_prompts.element_size(),
                "d2h_bytes_per_step": host_tokens.numel() * host_tokens.element_size()},
        "peak_mem_gb": 0.0 if on_cpu else torch.cuda.max_memory_allocated(dev) / 2**30,
    }
