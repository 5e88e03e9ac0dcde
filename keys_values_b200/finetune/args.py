"""Argument groups of the fine-tuning and evaluation commands; each dataclass is surfaced
on the command line as dotted flags (``--kv_cache.name``, ``--grad.layers_per_cell``, …).
Parity: ``keys_values/finetune/args.py:59-703``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

SUPPORTED_OPTIMIZERS = ("AdamW", "Adam", "SGD", "RMSprop", "Adagrad", "Adadelta", "Adamax")


@dataclass
class KVCacheArgs:
    """``name``: ``<policy>-<buffers>`` (see :class:`KVCacheFactory`); ``cache_length``: slots per
    layer; ``chunk_size``: tokens per chunk after the prefill; ``cache_kwargs``: passed to the
    cache constructor; ``randomize_chunk_sizes``: see ``create_chunk_sizes``; ``cpu_offload``:
    keep the quantized storage of inactive layers in pinned host memory."""

    name: str = "h2o-torch-quantized8"
    cache_length: int = 16384
    chunk_size: int = 1024
    cache_kwargs: Dict[str, Any] = field(default_factory=dict)
    randomize_chunk_sizes: bool = False
    allocate_buffers: bool = False
    max_num_ranges: Optional[int] = None
    cpu_offload: bool = False
    grace_period: int = 0
    max_chunk_size: Optional[int] = None
    attention_forward_temp_size_gb: Optional[float] = None

    def __post_init__(self):
        if self.cache_length <= 0 or self.chunk_size <= 0:
            raise ValueError("cache_length and chunk_size must be positive")

    def resolved_cache_kwargs(self) -> Dict[str, Any]:
        kw = dict(self.cache_kwargs)
        if "h2o" in self.name:
            kw.setdefault("max_chunk_size", self.max_chunk_size if self.max_chunk_size is not None else self.chunk_size)
            if self.grace_period:
                kw.setdefault("grace_period", self.grace_period)
        if self.max_num_ranges is not None:
            kw["max_num_ranges"] = self.max_num_ranges
        return kw


@dataclass
class GradientArgs:
    """``layers_per_cell``: layers per row of cells; ``chunks_per_cell_multiplier``: scales the
    cell length; ``single_tokens_for_targets``: schedule target tokens as chunks of one;
    ``layercp_qname / cachecp_qname``: optional quantization of layer-input / KV checkpoints;
    ``offload_checkpoints``: keep checkpoints in pinned host memory instead of device memory;
    ``save_attention_outputs``: keep attention outputs for the backward pass (None = auto);
    ``offload_weights``: the transformer blocks' weights live in pinned host memory and are streamed to the
    device block by block (``weight_slots`` device slots, default two per row of layers); the optimizer then
    updates the trainable block parameters on the host;
    ``profile_parts``: print a ``cProfile`` report (cumulative time) of the forward and / or backward part of the
    step; with ``profile_exit`` the process ends after the first report."""

    layers_per_cell: int = 1
    chunks_per_cell_multiplier: float = 1.0
    single_tokens_for_targets: bool = False
    use_new_cache: bool = True
    max_match_trials_pack_arg: Optional[int] = None
    layercp_qname: Optional[str] = None
    cachecp_qname: Optional[str] = None
    layercp_pin_memory: bool = True
    cachecp_pin_memory: bool = True
    offload_checkpoints: bool = False
    save_attention_outputs: Optional[bool] = None
    offload_weights: bool = False
    weight_slots: Optional[int] = None
    profile_parts: Optional[str] = None  # "forward" | "backward" | "both": cProfile report of that part of every step
    profile_exit: bool = False           # end the process after the first report


@dataclass
class OptimizerArgs:
    name: str = "AdamW"
    learning_rate: float = 2e-4
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    momentum: float = 0.0
    # master weights, fp32 gradients and optimizer moments in pinned host memory (finetune_offload_*)
    host_offload: bool = False

    def __post_init__(self):
        if self.name not in SUPPORTED_OPTIMIZERS:
            raise ValueError(f"optimizer {self.name} not supported; must be in {SUPPORTED_OPTIMIZERS}")

    def create(self, params):
        import torch

        cls = getattr(torch.optim, self.name)
        kw: Dict[str, Any] = dict(lr=self.learning_rate, weight_decay=self.weight_decay)
        if self.name in ("AdamW", "Adam", "Adamax"):
            kw.update(betas=(self.beta1, self.beta2), eps=self.eps)
        if self.name in ("SGD", "RMSprop"):
            kw.update(momentum=self.momentum)
        if self.host_offload:
            from keys_values_b200.optimize.host_optimizer import HostOffloadOptimizer

            return HostOffloadOptimizer(params, lambda host_params: cls(host_params, **kw))
        return cls(params, **kw)


@dataclass
class LoRAArgs:
    r: int = 8
    alpha: int = 16
    dropout: float = 0.05
    query: bool = True
    key: bool = False
    value: bool = True
    projection: bool = False
    mlp: bool = False
    head: bool = False
    kind: str = "default"

    def config_kwargs(self) -> Dict[str, Any]:
        return dict(lora_r=self.r, lora_alpha=self.alpha, lora_dropout=self.dropout, lora_query=self.query, lora_key=self.key,
                    lora_value=self.value, lora_projection=self.projection, lora_mlp=self.mlp, lora_head=self.head, lora_kind=self.kind)


@dataclass
class TrainArgs:
    save_interval: Optional[int] = 1000
    log_interval: int = 1
    global_batch_size: int = 8
    micro_batch_size: int = 1
    lr_warmup_steps: Optional[int] = 100
    lr_warmup_fraction: Optional[float] = None
    epochs: Optional[int] = None
    max_tokens: Optional[int] = None
    max_steps: Optional[int] = None
    max_seq_length: Optional[int] = None
    tie_embeddings: Optional[bool] = None
    max_norm: Optional[float] = None
    min_lr: float = 6e-5
    intermed_save_num: Optional[int] = 2

    def gradient_accumulation_iters(self, devices: int, num_nodes: int = 1) -> int:
        it = self.global_batch_size // (devices * num_nodes) // self.micro_batch_size
        assert it > 0, "global_batch_size must be at least devices * micro_batch_size"
        return it

    def warmup_iters(self, devices: int, max_iters: int, train_dataloader_len: int) -> int:
        if self.lr_warmup_fraction:
            return min(max_iters, int(self.lr_warmup_fraction * max_iters))
        if self.lr_warmup_steps:
            return min(max_iters, self.lr_warmup_steps * self.gradient_accumulation_iters(devices))
        return 0


@dataclass
class EvalArgs:
    interval: int = 100
    max_new_tokens: Optional[int] = 100
    max_iters: Optional[int] = 100
    initial_validation: bool = False
    final_validation: bool = True
    evaluate_example: str = "first"
    micro_batch_size: Optional[int] = None
    sample_metric: Optional[str] = None
    sample_metric_max_batches: Optional[int] = None
    generate_example: bool = True  # print a generated continuation of one validation prompt with every validation


@dataclass
class SDPAArgs:
    """Attention switches. This framework has one SDPA implementation per device (the native kernels
    on a GPU, a blocked PyTorch restatement elsewhere), so the back-end choices of the reference
    (``flex_attention``, ``flashinfer``, ``sdpa_kernels``, ``fused_*``) are accepted for command-line
    compatibility and have nothing to select. Two switches act:

    * ``use_eager_sdpa_always``: run the blocked PyTorch restatement on the GPU too (debugging,
      cross-checking the kernels on real data);
    * ``tmp_array_limit_gb``: largest score matrix the restatement forms at a time (it loops over
      blocks of query rows beyond it). Default 2 GB."""

    flex_attention: bool = False
    flashinfer: bool = False
    use_eager_sdpa_always: bool = False
    sdpa_kernels: Optional[List[str]] = None
    fused_rope: bool = True
    fused_rmsnorm: bool = True
    fused_swiglu: bool = True
    tmp_array_limit_gb: Optional[float] = None
