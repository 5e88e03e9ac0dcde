"""Programmatic training setup: model + caches + gradient model + optimizer.

This is the call a user makes to fine-tune with LoRA on long sequences without
going through the CLI (the CLI in :mod:`keys_values_b200.finetune.longcontext_lora`
builds on the same functions). Role of ``wrap_gpt_model`` and the inner part of
``fit`` in ``keys_values/finetune/longcontext_full.py:1055-1198``, ``:1493-1644``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Sequence

import torch

from keys_values_b200.kvcache.factory import KVCacheFactory, split_name
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.models import lora as lora_mod
from keys_values_b200.models.head_model import CrossEntropyOnLogits, HeadModel
from keys_values_b200.models.pos_encoding import position_encoding_factory
from keys_values_b200.utils.recovery import OOMRetry


@dataclass
class TrainingSetup:
    config: Any
    gpt_model: torch.nn.Module
    head_model: HeadModel
    model: LongContextGradientModel
    optimizer: torch.optim.Optimizer
    scheduler: Any = None
    grad_reducer: Any = None
    world_size: int = 1
    rank: int = 0
    max_norm: Optional[float] = None
    step: int = 0
    extras: Dict[str, Any] = field(default_factory=dict)


def create_lora_model(
    model_name: str,
    device,
    dtype,
    lora_r: int = 8,
    lora_alpha: int = 16,
    lora_dropout: float = 0.0,
    lora_targets: Sequence[str] = ("query", "key", "value", "projection"),
    lora_kind: str = "default",
    n_layer: Optional[int] = None,
    yarn_rope: bool = True,
    seed: int = 0,
    config_overrides: Optional[Dict[str, Any]] = None,
    tp_comm=None,
):
    """Random-init LoRA model on ``device`` (weights are loaded separately from a
    ``lit_model.pth`` with :func:`keys_values_b200.finetune.utils.load_model_checkpoint`). With ``tp_comm`` the
    model is this rank's shard (:class:`keys_values_b200.parallel.tp.TPLoRAGPT`); the returned configuration is
    the whole model's."""
    flags = {f"lora_{t}": True for t in lora_targets}
    over = dict(config_overrides or {})
    if n_layer is not None:
        over["n_layer"] = n_layer
    config = lora_mod.Config.from_name(
        model_name, lora_r=lora_r, lora_alpha=lora_alpha, lora_dropout=lora_dropout, lora_kind=lora_kind, **flags, **over
    )
    torch.manual_seed(seed)
    pos = position_encoding_factory(config, do_yarn=yarn_rope, device=device)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            if tp_comm is not None:
                from keys_values_b200.parallel.tp import TPLoRAGPT, local_config

                pos = position_encoding_factory(local_config(config, tp_comm.world), do_yarn=yarn_rope, device=device)
                model = TPLoRAGPT(config, tp_comm, pos_encoding=pos)
            else:
                model = lora_mod.GPT(config, pos_encoding=pos)
    finally:
        torch.set_default_dtype(prev)
    model.apply(model._init_weights)
    lora_mod.mark_only_lora_as_trainable(model)
    return config, model


def build_lora_training_setup(
    model_name: str,
    device,
    dtype=torch.bfloat16,
    cache_name: str = "h2o-torch-quantized8",
    cache_length: int = 16384,
    chunk_size: int = 1024,
    layers_per_cell: int = 1,
    lora_r: int = 8,
    lora_alpha: int = 16,
    lora_targets: Sequence[str] = ("query", "key", "value", "projection"),
    micro_batch_size: int = 1,
    n_layer: Optional[int] = None,
    world_size: int = 1,
    rank: int = 0,
    yarn_rope: bool = True,
    seed: int = 0,
    learning_rate: float = 2e-4,
    weight_decay: float = 0.0,
    max_norm: Optional[float] = 1.0,
    cache_kwargs: Optional[Dict[str, Any]] = None,
    grad_kwargs: Optional[Dict[str, Any]] = None,
    head_model: Optional[HeadModel] = None,
    overlap_allreduce: bool = True,
    train_all_parameters: bool = False,
    tp_size: int = 1,
    kv_cpu_offload: bool = False,
) -> TrainingSetup:
    """``train_all_parameters=True`` turns the set-up into a full fine-tune: every weight of the
    model (embeddings, norms, linears, head) is trainable, not only the LoRA factors.

    ``tp_size > 1``: the ``world_size`` ranks form ``world_size / tp_size`` data-parallel replicas of a model that
    is sharded over ``tp_size`` consecutive ranks (heads, KV heads and MLP columns; every rank keeps the caches and
    the eviction state of its KV heads). Ranks of one replica must be fed the same batch; ``seed`` must then be
    the same on all ranks (replicated parameters are initialised from it)."""
    tp_comm, dp_group, dp_world, dp_rank = None, None, world_size, rank
    if tp_size > 1:
        import torch.distributed as dist

        from keys_values_b200.parallel.tp import TPComm

        if world_size % tp_size:
            raise ValueError(f"world_size = {world_size} must be a multiple of tp_size = {tp_size}")
        dp_world, dp_rank, tp_rank = world_size // tp_size, rank // tp_size, rank % tp_size
        tp_group = None
        for k in range(dp_world):  # every rank creates every group, in the same order
            grp = dist.new_group(list(range(k * tp_size, (k + 1) * tp_size)))
            if k == dp_rank:
                tp_group = grp
        for k in range(tp_size):
            grp = dist.new_group(list(range(k, world_size, tp_size)))
            if k == tp_rank:
                dp_group = grp
        tp_comm = TPComm(tp_size, tp_rank, device, group=tp_group, dtype=dtype)
    config, gpt = create_lora_model(
        model_name, device, dtype, lora_r=lora_r, lora_alpha=lora_alpha, lora_targets=lora_targets,
        n_layer=n_layer, yarn_rope=yarn_rope, seed=seed, tp_comm=tp_comm,
    )
    if train_all_parameters:
        for p in gpt.parameters():
            p.requires_grad_(True)
    ck = dict(cache_kwargs or {})
    cname, _ = split_name(cache_name)
    if "h2o" in cname and "max_chunk_size" not in ck:
        ck["max_chunk_size"] = chunk_size
    if kv_cpu_offload:  # quantized storage of all layers in pinned host memory, one layer at a time on the device
        caches, offloader = KVCacheFactory.create_cpu_offloading(gpt, cache_name, micro_batch_size, cache_length, device=device, dtype=dtype,
                                                                 cache_kwargs=ck)
        gpt._kv_offloader = offloader
    else:
        caches = KVCacheFactory.create(gpt, cache_name, micro_batch_size, cache_length, device=device, dtype=dtype, cache_kwargs=ck)
    gpt.assign_kv_caches(caches)
    head = head_model if head_model is not None else CrossEntropyOnLogits(config)
    model = LongContextGradientModel(gpt, head, layers_per_cell=layers_per_cell, chunk_size=chunk_size, **(grad_kwargs or {}))
    model.train()
    params = [p for p in gpt.parameters() if p.requires_grad] + [p for p in head.parameters() if p.requires_grad]
    optimizer = torch.optim.AdamW(params, lr=learning_rate, weight_decay=weight_decay, fused=torch.device(device).type == "cuda")
    setup = TrainingSetup(config, gpt, head, model, optimizer, world_size=world_size, rank=rank, max_norm=max_norm)
    if tp_comm is not None:
        setup.extras.update(tp_comm=tp_comm, dp_group=dp_group, dp_world=dp_world, dp_rank=dp_rank)
    if dp_world > 1:
        from keys_values_b200.parallel.dp import GradientReducer

        setup.grad_reducer = GradientReducer(params, world_size=dp_world, rank=dp_rank, device=device, overlap=overlap_allreduce,
                                             group=dp_group)
        if overlap_allreduce:
            model.row_done_hook = setup.grad_reducer.row_done_hook(gpt)
    return setup


def _free_after_oom(setup: TrainingSetup) -> None:
    import gc

    setup.model.clear()  # checkpoints, replay logs and saved attention outputs of the failed attempt
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def check_native_status(setup: TrainingSetup, device) -> None:
    """Reads the device status word before the optimizer may use the gradients of this step. A kernel
    whose bounded wait ran out returns without doing its work (gradients not reduced, a tile not
    computed); stepping on that would let the replicas diverge silently. Raises ``RankFailure`` (data
    parallel) or ``NativeError`` and marks this rank as failed for its peers."""
    device = torch.device(device)
    if device.type != "cuda":
        return
    try:
        if setup.grad_reducer is not None:
            setup.grad_reducer.check()
        else:
            from keys_values_b200.ops import cuda as _cu

            _cu.check_status(device)
    except Exception as ex:
        health = setup.extras.get("health")
        if health is not None:
            health.mark_failed(f"{type(ex).__name__}: {ex}")
        raise


def training_step(setup: TrainingSetup, input_ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Forward, backward, gradient all-reduce (mean over ranks), clipping, optimizer
    step. Returns the (local) loss as a 0-d device tensor."""
    health = setup.extras.get("health")
    if health is not None:
        # host rendezvous: no rank launches the collectives of a step that a lost peer will never join
        health.enter_step(setup.step, grace_s=setup.extras.get("health_grace_s", 60.0))

    def attempt(_limit_gb: float, save_attention: bool):
        if not save_attention:
            setup.model.save_attention_outputs = False  # recompute in the backward pass instead
        setup.optimizer.zero_grad(set_to_none=False if setup.grad_reducer is not None else True)
        if setup.grad_reducer is not None:
            setup.grad_reducer.begin_step()
        out = setup.model(input_ids, targets)
        out.backward()
        return out

    if setup.world_size == 1:
        # out of memory: free, give up the saved attention outputs, retry (single rank only: with
        # several ranks a retry on one of them would leave the others inside the gradient all-reduce)
        loss = OOMRetry(limits_gb=(0.0,), free_fn=lambda: _free_after_oom(setup)).run(attempt)
    else:
        loss = attempt(0.0, True)
    if setup.grad_reducer is not None:
        setup.grad_reducer.finish_step()
    check_native_status(setup, input_ids.device)
    if setup.max_norm is not None:
        if setup.extras.get("tp_comm") is not None:
            from keys_values_b200.parallel.tp import clip_grad_norm_sharded

            clip_grad_norm_sharded(setup.gpt_model, setup.max_norm)
        else:
            params = [p for g in setup.optimizer.param_groups for p in g["params"] if p.grad is not None]
            torch.nn.utils.clip_grad_norm_(params, setup.max_norm)
    setup.optimizer.step()
    if setup.scheduler is not None:
        setup.scheduler.step()
    setup.step += 1
    return loss.detach()
