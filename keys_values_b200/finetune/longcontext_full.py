"""Long-context fine-tuning driver (full weights or LoRA).

``setup`` validates the arguments and launches one process per GPU; ``main`` builds model,
caches, gradient model, optimizer and data; ``fit`` is the training loop: chunked forward,
cell-wise backward, gradient all-reduce over ranks (overlapped with the backward), gradient
clipping, optimizer step, logging, periodic validation and checkpoints with resumable
training state. Parity: ``keys_values/finetune/longcontext_full.py:153-2008``.
"""
from __future__ import annotations

import dataclasses
import math
import os
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist

from keys_values_b200.config import Config
from keys_values_b200.data.base import DataModule
from keys_values_b200.data.dataloader import CycleIterator
from keys_values_b200.finetune import utils as fu
from keys_values_b200.finetune.args import EvalArgs, GradientArgs, KVCacheArgs, LoRAArgs, OptimizerArgs, SDPAArgs, TrainArgs
from keys_values_b200.finetune.batch_transform import BatchTransformFactory
from keys_values_b200.finetune.resume_state import TrainingStateManager, find_resume_dir, restore_from_training_state
from keys_values_b200.kvcache.consts import split_name
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.models.head_model import CrossEntropyOnLogits, HeadModelFactory
from keys_values_b200.models.pos_encoding import position_encoding_factory
from keys_values_b200.utils import get_default_supported_precision, message_memory_all_devices, num_parameters, str_to_torch_dtype


@dataclasses.dataclass
class TrainingStateVars:
    iter_num: int = 0
    step_count: int = 0
    total_tokens: int = 0
    train_time: float = 0.0
    saved_dirs: List[str] = dataclasses.field(default_factory=list)


def _dist_info():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def setup(
    checkpoint_dir: Union[str, Path],
    out_dir: Union[str, Path] = Path("out/finetune/long-full"),
    precision: Optional[str] = None,
    devices: int = 1,
    resume: Union[bool, str, Path] = False,
    data: Optional[DataModule] = None,
    train: TrainArgs = TrainArgs(),
    eval: EvalArgs = EvalArgs(),
    optimizer: OptimizerArgs = OptimizerArgs(),
    kv_cache: KVCacheArgs = KVCacheArgs(),
    grad: GradientArgs = GradientArgs(),
    sdpa: SDPAArgs = SDPAArgs(),
    lora: Optional[LoRAArgs] = None,
    head_model: str = CrossEntropyOnLogits.NAME,
    head_model_kwargs: Optional[Dict[str, Any]] = None,
    logger_name: str = "csv",
    seed: int = 1337,
    yarn_rope: bool = True,
    model_name: Optional[str] = None,
    profile_grad_times: int = 0,
    record_gpu_memory_snapshots: Optional[int] = None,
    tp: int = 1,
) -> None:
    """Entry point of ``finetune_long_full`` (and, with ``lora`` given, ``finetune_long_lora``).
    ``tp > 1``: the ``devices`` ranks form ``devices / tp`` data-parallel replicas of a model sharded over ``tp``
    consecutive ranks (heads, KV heads, MLP columns); checkpoints are written for the whole model.
    ``checkpoint_dir`` holds ``lit_model.pth`` and ``model_config.yaml``; with ``model_name`` the
    architecture is taken from the registry and weights are initialised randomly if no
    ``lit_model.pth`` is present."""
    from keys_values_b200.parallel.launch import launch

    checkpoint_dir, out_dir = Path(checkpoint_dir), Path(out_dir)
    if not HeadModelFactory.is_supported(head_model):
        raise ValueError(f"head_model = {head_model} not supported")
    split_name(kv_cache.name)  # validates the cache name
    if devices < 1:
        raise ValueError("devices must be >= 1")
    if tp < 1 or devices % tp:
        raise ValueError(f"devices = {devices} must be a multiple of tp = {tp}")
    if tp > 1 and (grad.offload_weights or optimizer.host_offload):
        raise ValueError("tensor parallelism does not combine with host-resident weights or optimizer state")
    precision = precision or get_default_supported_precision(training=True)
    hparams = dict(checkpoint_dir=str(checkpoint_dir), out_dir=str(out_dir), precision=precision, devices=devices, train=train, eval=eval,
                   optimizer=optimizer, kv_cache=kv_cache, grad=grad, sdpa=sdpa, lora=lora, head_model=head_model, seed=seed,
                   yarn_rope=yarn_rope, model_name=model_name, tp=tp)
    launch(main, devices, tp=tp, checkpoint_dir=checkpoint_dir, out_dir=out_dir, precision=precision, resume=resume, data=data, train=train,
           eval=eval, optimizer=optimizer, kv_cache=kv_cache, grad=grad, sdpa=sdpa, lora=lora, head_model_name=head_model,
           head_model_kwargs=head_model_kwargs or {}, logger_name=logger_name, seed=seed, yarn_rope=yarn_rope, model_name=model_name,
           hparams=hparams, profile_grad_times=profile_grad_times, record_gpu_memory_snapshots=record_gpu_memory_snapshots)


def create_gpt_model(checkpoint_dir: Path, model_name: Optional[str], lora: Optional[LoRAArgs], device, dtype, yarn_rope: bool, tp_comm=None):
    """Returns ``(config of the whole model, model)``; with ``tp_comm`` the model is this rank's shard."""
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.models.model import GPT

    kwargs = lora.config_kwargs() if lora is not None else {}
    cfg_cls = lora_mod.Config if lora is not None else Config
    if (Path(checkpoint_dir) / "model_config.yaml").is_file():
        config = cfg_cls.from_file(Path(checkpoint_dir) / "model_config.yaml", **kwargs)
    elif model_name is not None:
        config = cfg_cls.from_name(model_name, **kwargs)
    else:
        raise FileNotFoundError(f"{checkpoint_dir}/model_config.yaml not found and no model_name given")
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            if tp_comm is not None:
                from keys_values_b200.parallel import tp as tp_mod

                pos = position_encoding_factory(tp_mod.local_config(config, tp_comm.world), do_yarn=yarn_rope, device=device)
                model = (tp_mod.TPLoRAGPT if lora is not None else tp_mod.TPGPT)(config, tp_comm, pos_encoding=pos)
            else:
                pos = position_encoding_factory(config, do_yarn=yarn_rope, device=device)
                model = (lora_mod.GPT if lora is not None else GPT)(config, pos_encoding=pos)
    finally:
        torch.set_default_dtype(prev)
    model.apply(model._init_weights)
    if lora is not None:
        lora_mod.mark_only_lora_as_trainable(model)
    return config, model


def wrap_gpt_model(gpt_model, head_model, kv_cache: KVCacheArgs, grad: GradientArgs, micro_batch_size: int, device, dtype,
                   profile_steps: bool = False, weight_grad_reduce_fn=None) -> LongContextGradientModel:
    """Create the KV caches (optionally with host offload of the quantized storage), assign
    them to the model, and wrap model + head into the gradient model."""
    ck = kv_cache.resolved_cache_kwargs()
    if kv_cache.cpu_offload:
        caches, offloader = KVCacheFactory.create_cpu_offloading(gpt_model, kv_cache.name, micro_batch_size, kv_cache.cache_length,
                                                                 device=device, dtype=dtype, cache_kwargs=ck)
        gpt_model._kv_offloader = offloader
    else:
        caches = KVCacheFactory.create(gpt_model, kv_cache.name, micro_batch_size, kv_cache.cache_length, device=device, dtype=dtype,
                                       cache_kwargs=ck)
    gpt_model.assign_kv_caches(caches)
    model = LongContextGradientModel(
        gpt_model, head_model, layers_per_cell=grad.layers_per_cell, chunk_size=kv_cache.chunk_size,
        randomize_chunk_sizes=kv_cache.randomize_chunk_sizes, chunks_per_cell_multiplier=grad.chunks_per_cell_multiplier,
        single_tokens_for_targets=grad.single_tokens_for_targets, offload_checkpoints=grad.offload_checkpoints,
        pin_memory=grad.layercp_pin_memory, layercp_qname=grad.layercp_qname, cachecp_qname=grad.cachecp_qname,
        save_attention_outputs=grad.save_attention_outputs, profile_steps=profile_steps,
        profile_parts=grad.profile_parts, profile_exit=grad.profile_exit,
    )
    if grad.offload_weights:
        from keys_values_b200.optimize.weight_streaming import WeightStreamer

        model.weight_streamer = WeightStreamer(gpt_model, device, n_slots=grad.weight_slots or 2 * grad.layers_per_cell,
                                               reduce_fn=weight_grad_reduce_fn)
    return model


def apply_sdpa_args(sdpa: Optional[SDPAArgs], rank: int = 0) -> None:
    """Puts the two acting switches of :class:`SDPAArgs` into effect and says which of the others were given
    although they select nothing here."""
    from keys_values_b200 import ops

    sdpa = sdpa if sdpa is not None else SDPAArgs()
    ops.set_native_attention(not sdpa.use_eager_sdpa_always)
    ops.set_tmp_array_limit_gb(sdpa.tmp_array_limit_gb)
    ignored = [n for n in ("flex_attention", "flashinfer") if getattr(sdpa, n)] + (["sdpa_kernels"] if sdpa.sdpa_kernels else [])
    if ignored and rank == 0:
        print(f"sdpa: {', '.join(ignored)} given; this framework has one attention implementation per device, nothing is selected")
    if sdpa.use_eager_sdpa_always and rank == 0:
        print("sdpa: attention runs in the blocked PyTorch restatement on every device (use_eager_sdpa_always)")


def main(rank: int, local_rank: int, world_size: int, *, checkpoint_dir, out_dir, precision, resume, data, train, eval, optimizer, kv_cache,
         grad, sdpa=None, lora, head_model_name, head_model_kwargs, logger_name, seed, yarn_rope, model_name, hparams, profile_grad_times,
         record_gpu_memory_snapshots, tp: int = 1) -> None:
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dtype = str_to_torch_dtype(precision)
    apply_sdpa_args(sdpa, rank)
    torch.manual_seed(seed)
    out_dir = Path(out_dir)
    if rank == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
    logger = fu.choose_logger(logger_name, out_dir) if rank == 0 else None
    # layout of the ranks: dp_world replicas of a model sharded over tp consecutive ranks
    tp_comm, dp_group, dp_world, dp_rank = None, None, world_size, rank
    if tp > 1:
        from keys_values_b200.parallel.tp import TPComm

        dp_world, dp_rank, tp_rank = world_size // tp, rank // tp, rank % tp
        tp_group = None
        for k in range(dp_world):  # every rank creates every group, in the same order
            grp = dist.new_group(list(range(k * tp, (k + 1) * tp)))
            tp_group = grp if k == dp_rank else tp_group
        for k in range(tp):
            grp = dist.new_group(list(range(k, world_size, tp)))
            dp_group = grp if k == tp_rank else dp_group
        tp_comm = TPComm(tp, tp_rank, device, group=tp_group, dtype=dtype)
    config, gpt_model = create_gpt_model(checkpoint_dir, model_name, lora, device, dtype, yarn_rope, tp_comm=tp_comm)
    head_model = HeadModelFactory.create(head_model_name, config, **head_model_kwargs).to(device)
    resume_dir = find_resume_dir(out_dir, resume)
    fu.load_model_checkpoint(gpt_model, checkpoint_dir, resume_dir, head_model)
    reduce_fn = None
    if world_size > 1:
        def reduce_fn(flat: torch.Tensor) -> None:  # streamed blocks: mean over ranks before the gradients leave for the host
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            flat.mul_(1.0 / world_size)
    model = wrap_gpt_model(gpt_model, head_model, kv_cache, grad, train.micro_batch_size, device, dtype, profile_steps=profile_grad_times > 0,
                           weight_grad_reduce_fn=reduce_fn)
    if rank == 0:
        print(f"trainable parameters: {num_parameters(gpt_model, True):,} of {num_parameters(gpt_model):,}")
    params = [p for p in gpt_model.parameters() if p.requires_grad] + [p for p in head_model.parameters() if p.requires_grad]
    if grad.offload_weights and optimizer.host_offload:
        # the streamed blocks' parameters already live on the host and are updated there; the optimizer keeps its
        # state next to each parameter (host for the blocks, device for embedding and head)
        optimizer = dataclasses.replace(optimizer, host_offload=False)
    opt = optimizer.create(params)
    # data
    tokenizer = None
    if (Path(checkpoint_dir) / "tokenizer.json").is_file() or (Path(checkpoint_dir) / "tokenizer.model").is_file():
        from keys_values_b200.tokenizer import Tokenizer

        tokenizer = Tokenizer(checkpoint_dir)
    if data is None:
        from keys_values_b200.data.module import SyntheticLongContext

        data = SyntheticLongContext(config.vocab_size, seq_lengths=(4 * kv_cache.cache_length,), num_targets=kv_cache.chunk_size)
    # the ranks of a replica read the same batches
    data.connect(tokenizer=tokenizer, batch_size=train.micro_batch_size, max_seq_length=train.max_seq_length, num_devices=dp_world, rank=dp_rank)
    if rank == 0:
        data.prepare_data()
    if world_size > 1:
        dist.barrier()
    data.setup()
    train_loader, val_loader = data.train_dataloader(), data.val_dataloader()
    accum = train.gradient_accumulation_iters(dp_world)
    steps_per_epoch = max(1, len(train_loader) // accum)
    max_steps = train.max_steps or (train.epochs or 1) * steps_per_epoch
    warmup = min(max_steps, train.lr_warmup_steps or int((train.lr_warmup_fraction or 0.0) * max_steps))
    scheduler = fu.get_lr_scheduler(getattr(opt, "optimizer", opt), warmup_steps=warmup, max_steps=max_steps, min_lr=train.min_lr)
    state = TrainingStateVars()
    if resume_dir is not None:
        st = restore_from_training_state(resume_dir, opt, scheduler, rank, world_size, tp_rank=rank % tp if tp > 1 else None)
        state.iter_num, state.step_count = st["iter_num"], st["step_count"]
        if hasattr(train_loader, "load_state_dict"):
            train_loader.load_state_dict(st.get("iterator", {}))
    grad_reducer = None
    if dp_world > 1:
        from keys_values_b200.parallel.dp import GradientReducer

        resident = [p for p in params if p.device.type == device.type]  # streamed blocks reduce their own gradients
        grad_reducer = GradientReducer(resident, world_size=dp_world, rank=dp_rank, device=device, group=dp_group) if resident else None
        if grad_reducer is not None:
            model.row_done_hook = grad_reducer.row_done_hook(gpt_model)
    pad_id = getattr(tokenizer, "pad_id", None) or 0
    batch_transform = BatchTransformFactory.from_head_model(head_model_name, pad_id=pad_id)
    fit(model=model, optimizer=opt, scheduler=scheduler, train_loader=train_loader, val_loader=val_loader, batch_transform=batch_transform,
        train=train, eval=eval, state=state, max_steps=max_steps, accum=accum, device=device, rank=rank, world_size=world_size,
        grad_reducer=grad_reducer, logger=logger, out_dir=out_dir, checkpoint_dir=Path(checkpoint_dir), lora=lora is not None,
        hparams=hparams, profile_grad_times=profile_grad_times, record_gpu_memory_snapshots=record_gpu_memory_snapshots, tokenizer=tokenizer,
        dp_world=dp_world, tp=tp)
    final = out_dir / "final"
    fu.save_model_checkpoint(gpt_model, head_model, final, lora=lora is not None, rank=rank)  # a collective under tensor parallelism
    if rank == 0:
        fu.copy_config_files(Path(checkpoint_dir), final)
        config.save(final / "model_config.yaml")
        fu.save_hyperparameters(hparams, final)
        report = fu.finetuning_performance_report(state.train_time, state.total_tokens, state.step_count, device, out_dir)
        print("performance report: " + ", ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in report.items()))
        print(message_memory_all_devices("memory: "))


def _all_reduce_mean(x: torch.Tensor, world_size: int) -> torch.Tensor:
    if world_size > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM)
        x = x / world_size
    return x


@torch.no_grad()
def validate(model: LongContextGradientModel, val_loader, batch_transform, device, max_iters: Optional[int]) -> torch.Tensor:
    model.eval()
    losses = []
    for k, batch in enumerate(val_loader):
        if max_iters is not None and k >= max_iters:
            break
        b = batch_transform(batch)
        loss = model(b["input_ids"].to(device), b["targets"].to(device))
        losses.append(loss.float().mean())
    model.train()
    return torch.stack(losses).mean() if losses else torch.tensor(float("nan"), device=device)


def validate_sample_metric(model, val_loader, tokenizer, device, eval: EvalArgs, world_size: int) -> Dict[str, float]:
    """Generate answers for validation batches and score them (``eval.sample_metric``)
    (``keys_values/finetune/longcontext_full.py:1880-1903``)."""
    from keys_values_b200.evaluation.evaluator import sample_metric_on_loader

    gpt = model.gpt_model
    width = gpt.max_seq_length
    try:
        res = sample_metric_on_loader(gpt, tokenizer, val_loader, eval.sample_metric, device, eval.sample_metric_max_batches,
                                      eval.max_new_tokens or 64, model.chunk_size, getattr(tokenizer, "pad_id", None) or 0)
    finally:
        gpt.reset()
        gpt.max_seq_length = width
    mean = _all_reduce_mean(torch.tensor(res["mean"], device=device), world_size)
    return {f"val_{eval.sample_metric}": float(mean)}


def validate_and_all_reduce(model, val_loader, batch_transform, device, eval: EvalArgs, world_size: int, tokenizer=None) -> Dict[str, float]:
    t0 = time.perf_counter()
    val_loss = validate(model, val_loader, batch_transform, device, eval.max_iters)
    val_loss = _all_reduce_mean(val_loss.to(device), world_size)
    v = float(val_loss)
    from keys_values_b200 import ops as _ops

    _ops.check_status(device)  # the loss has just been read: a kernel that gave up during validation is reported here
    metrics = {"val_loss": v, "val_ppl": math.exp(v) if v < 50 else float("inf")}
    if eval.sample_metric is not None and tokenizer is not None:
        metrics.update(validate_sample_metric(model, val_loader, tokenizer, device, eval, world_size))
    metrics["val_time"] = time.perf_counter() - t0
    return metrics


def save_checkpoint_regular(model: LongContextGradientModel, out_dir: Path, step: int, checkpoint_dir: Path, lora: bool, hparams, rank: int,
                            state: TrainingStateVars, intermed_save_num: Optional[int]) -> Path:
    step_dir = out_dir / f"step-{step:06d}"
    fu.save_model_checkpoint(model.gpt_model, model.head_model, step_dir, lora=lora, rank=rank)  # a collective under tensor parallelism
    if rank == 0:
        fu.copy_config_files(checkpoint_dir, step_dir)
        getattr(model.gpt_model, "full_config", model.gpt_model.config).save(step_dir / "model_config.yaml")
        fu.save_hyperparameters(hparams, step_dir)
        state.saved_dirs.append(str(step_dir))
        if intermed_save_num is not None:
            import shutil

            while len(state.saved_dirs) > intermed_save_num:
                shutil.rmtree(state.saved_dirs.pop(0), ignore_errors=True)
    return step_dir


def fit(*, model, optimizer, scheduler, train_loader, val_loader, batch_transform, train: TrainArgs, eval: EvalArgs, state: TrainingStateVars,
        max_steps: int, accum: int, device, rank: int, world_size: int, grad_reducer, logger, out_dir: Path, checkpoint_dir: Path, lora: bool,
        hparams, profile_grad_times: int = 0, record_gpu_memory_snapshots: Optional[int] = None, tokenizer=None,
        dp_world: Optional[int] = None, tp: int = 1) -> None:
    """``world_size`` ranks in ``dp_world`` replicas (default: every rank is a replica) of ``tp`` shards each."""
    from keys_values_b200.utils.recovery import OOMRetry

    dp_world = world_size if dp_world is None else dp_world
    ts_manager = TrainingStateManager(out_dir, rank, world_size, tp_rank=rank % tp if tp > 1 else None)
    train_iter = CycleIterator(train_loader)
    throughput = fu.ThroughputMonitor(dp_world)
    samples_seen = 0

    def free_after_oom() -> None:
        import gc

        model.clear()  # checkpoints, replay logs and saved attention outputs of the failed attempt
        gc.collect()
        if device.type == "cuda":
            torch.cuda.empty_cache()

    def show_example() -> None:
        if not (eval.generate_example and rank == 0 and val_loader is not None):
            return
        try:
            batch = batch_transform(next(iter(val_loader)))
        except StopIteration:
            return
        ids = batch["input_ids"][0]
        n_t = batch["targets"].shape[1]
        prompt = ids[: max(1, ids.numel() - n_t + 1)]
        text = fu.generate_example(model.gpt_model, tokenizer, prompt, min(eval.max_new_tokens or 32, 64), model.chunk_size, device)
        print(f"example continuation ({prompt.numel()} prompt tokens): {text}")

    if eval.initial_validation:
        metrics = validate_and_all_reduce(model, val_loader, batch_transform, device, eval, world_size, tokenizer)
        if rank == 0:
            print(f"initial validation: {metrics}")
            logger.log_dict(metrics, step=state.step_count)
    recorder = None
    if record_gpu_memory_snapshots:
        from keys_values_b200.tools.gpu_memory import RecordGPUMemory

        recorder = RecordGPUMemory(out_dir / "gpu_memory", max_entries=record_gpu_memory_snapshots)
    if world_size > 1:
        dist.barrier()
    params = [p for g in optimizer.param_groups for p in g["params"]]
    while state.step_count < max_steps:
        t0 = time.perf_counter()
        if grad_reducer is not None:
            grad_reducer.begin_step()
            grad_reducer.flat.zero_()
        else:
            optimizer.zero_grad(set_to_none=True)
        if getattr(model, "weight_streamer", None) is not None:
            model.weight_streamer.zero_grad()
        step_loss = torch.zeros((), device=device)
        step_tokens = 0
        if recorder is not None:
            recorder.start(f"step{state.step_count}")
        for micro in range(accum):
            batch = batch_transform(next(train_iter))
            ids, targets = batch["input_ids"].to(device, non_blocking=True), batch["targets"].to(device, non_blocking=True)
            # token-weighted averaging over ranks: weight this rank's loss by its share of target tokens
            n_tok = (targets != -100).sum().float()
            scale = 1.0 / accum
            if world_size > 1:
                mean_tok = _all_reduce_mean(n_tok.clone(), world_size)
                scale = scale * float(n_tok / mean_tok.clamp(min=1))
            if grad_reducer is not None and micro < accum - 1:
                hook, model.row_done_hook = model.row_done_hook, None  # reduce only after the last micro-batch

            def attempt(_limit_gb: float, save_attention: bool):
                if not save_attention:
                    model.save_attention_outputs = False  # recompute in the backward pass instead
                out = model(ids, targets, scale_factor=scale)
                out.backward()
                return out

            if world_size == 1:
                # out of memory in the forward or backward pass: free, give up the saved attention outputs, retry
                # (one rank only: with several, a retry on one of them would leave the others in the all-reduce)
                loss = OOMRetry(limits_gb=(0.0,), free_fn=free_after_oom, verbose=True).run(attempt)
            else:
                loss = attempt(0.0, True)
            if grad_reducer is not None and micro < accum - 1:
                model.row_done_hook = hook
            step_loss += loss.detach().float()
            step_tokens += ids.numel()
            samples_seen += ids.shape[0]
            state.iter_num += 1
        if grad_reducer is not None:
            grad_reducer.finish_step()
            grad_reducer.check()  # raises RankFailure if a wait of the all-reduce ran out: no step on unreduced gradients
        elif device.type == "cuda":
            from keys_values_b200.ops import cuda as _cu

            _cu.check_status(device)
        if recorder is not None:
            recorder.stop()
        if train.max_norm is not None:
            if tp > 1:  # the norm of the whole model: sharded tensors summed over the ranks, replicated ones counted once
                from keys_values_b200.parallel.tp import clip_grad_norm_sharded

                clip_grad_norm_sharded(model.gpt_model, train.max_norm)
            elif hasattr(optimizer, "clip_grad_norm_"):  # gradients are clipped where the optimizer lives (host)
                optimizer.clip_grad_norm_(train.max_norm)
            else:
                torch.nn.utils.clip_grad_norm_([p for p in params if p.grad is not None], train.max_norm)
        optimizer.step()
        scheduler.step()
        state.step_count += 1
        step_loss = _all_reduce_mean(step_loss, world_size)
        state.total_tokens += step_tokens * dp_world
        dt = time.perf_counter() - t0
        state.train_time += dt
        if rank == 0 and state.step_count % train.log_interval == 0:
            metrics = {"loss": float(step_loss), "iter": state.iter_num, "step": state.step_count, "epoch": train_iter.epoch,
                       "iter_time": dt, "tokens": step_tokens * dp_world, "total_tokens": state.total_tokens,
                       "tokens_per_sec": step_tokens * dp_world / dt, "learning_rate": scheduler.get_last_lr()[0]}
            throughput.update(time=state.train_time, batches=state.iter_num, samples=samples_seen, lengths=state.total_tokens // dp_world)
            metrics.update(throughput.compute())
            logger.log_dict(metrics, step=state.step_count)
            print(f"step {state.step_count}/{max_steps} | loss {metrics['loss']:.4f} | {dt:.1f} s | {metrics['tokens_per_sec']:.0f} tok/s")
        if profile_grad_times and state.step_count >= profile_grad_times:
            if rank == 0:
                import csv

                with open(out_dir / "profile_grad_times.csv", "w", newline="") as fp:
                    recs = model.profile_records
                    w = csv.DictWriter(fp, fieldnames=sorted({k for r in recs for k in r}))
                    w.writeheader()
                    w.writerows(recs)
            return
        if eval.interval and state.step_count % eval.interval == 0:
            metrics = validate_and_all_reduce(model, val_loader, batch_transform, device, eval, world_size, tokenizer)
            if rank == 0:
                logger.log_dict(metrics, step=state.step_count)
                print(f"validation: {metrics}")
            show_example()
            if world_size > 1:
                dist.barrier()
        if train.save_interval and state.step_count % train.save_interval == 0:
            step_dir = save_checkpoint_regular(model, out_dir, state.step_count, checkpoint_dir, lora, hparams, rank, state, train.intermed_save_num)
            it_state = train_loader.state_dict() if hasattr(train_loader, "state_dict") else {}
            ts_manager.save(step_dir, optimizer, scheduler, state.iter_num, state.step_count, None, it_state)
            if world_size > 1:
                dist.barrier()
    if eval.final_validation:
        metrics = validate_and_all_reduce(model, val_loader, batch_transform, device, eval, world_size, tokenizer)
        if rank == 0:
            logger.log_dict(metrics, step=state.step_count)
            print(f"final validation: {metrics}")


def inherit_cli_signature(fn, defaults: Optional[Dict[str, Any]] = None):
    """Give a thin ``setup(**kwargs)`` variant the parameters of :func:`setup` (with other
    defaults), so that the command line parser sees the same flags."""
    import inspect

    sig = inspect.signature(setup)
    params = []
    for name, p in sig.parameters.items():
        if defaults and name in defaults:
            p = p.replace(default=defaults[name])
        params.append(p)
    fn.__signature__ = sig.replace(parameters=params)
    import typing

    fn.__annotations__ = typing.get_type_hints(setup)
    return fn
