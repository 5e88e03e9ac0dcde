"""LoRA / DoRA variants of the model.

``y = x Wᵀ + (α/r) · drop(x) Aᵀ Bᵀ`` on any of q/k/v, attention projection, MLP
and head. Parameter names and shapes follow LitGPT (``lora_A (r·n_enabled, in)``,
``lora_B (Σ enabled out, r)``, pretrained weights under ``.linear.``), so that
``lit_model.pth`` and ``lit_model.lora.pth`` files are interchangeable. Parity:
``keys_values/lora.py:44-443``, ``lora_utils.py:74-339``, ``dora_utils.py:32-193``.

``lora_kind``: ``default`` (standard), ``rms_norm`` (RMSNorm on the LoRA branch),
``dora`` (weight-decomposed: the merged weight is renormalised by detached row
norms times learnable ``lora_scales``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Type, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from keys_values_b200.config import Config as BaseConfig
from keys_values_b200.models import model as base
from keys_values_b200.models.model import RMSNorm


@dataclass
class Config(BaseConfig):
    lora_r: int = 0
    lora_alpha: int = 1
    lora_dropout: float = 0.0
    lora_query: bool = False
    lora_key: bool = False
    lora_value: bool = False
    lora_projection: bool = False
    lora_mlp: bool = False
    lora_head: bool = False
    lora_kind: str = "default"

    def __post_init__(self):
        super().__post_init__()
        if self.lora_kind not in ("default", "rms_norm", "dora"):
            raise ValueError(f"lora_kind = {self.lora_kind} must be 'default', 'rms_norm' or 'dora'")

    @property
    def mlp_class(self) -> Type:
        import keys_values_b200.models.lora as _l

        return getattr(_l, self.mlp_class_name)


def row_lengths(w: torch.Tensor, eps: float) -> torch.Tensor:
    return torch.sqrt(w.float().pow(2).sum(dim=1) + eps)


class LoRALinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, r: int = 0, lora_alpha: int = 1, lora_dropout: float = 0.0,
                 use_rms_norm: bool = False, **kwargs):
        super().__init__()
        self.r, self.lora_alpha = r, lora_alpha
        self.lora_dropout = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        self.merged = False
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        self.rms_norm = None
        if r > 0:
            self.lora_A = nn.Parameter(torch.empty((r, in_features)))
            self.lora_B = nn.Parameter(torch.empty((out_features, r)))
            self.scaling = lora_alpha / r
            if use_rms_norm:
                self.rms_norm = RMSNorm(out_features)
            self.reset_parameters()

    @property
    def weight(self) -> torch.Tensor:
        return self.linear.weight

    @property
    def bias(self):
        return self.linear.bias

    def reset_parameters(self) -> None:
        if hasattr(self, "lora_A"):
            nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B)

    def get_lora_AB(self) -> torch.Tensor:
        """``ΔW = (α/r) · B A`` with the shape of the pretrained weight."""
        return (self.lora_B @ self.lora_A) * self.scaling

    def merge(self) -> None:
        if self.r > 0 and not self.merged and self.rms_norm is None:
            self.linear.weight.data += self.get_lora_AB().to(self.linear.weight.dtype)
            self.merged = True

    def _lora_branch(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(F.linear(self.lora_dropout(x), self.lora_A), self.lora_B) * self.scaling

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.r == 0 or self.merged:
            return self.linear(x)
        if self.rms_norm is None:
            # pretrained + scaling · (x A^T) B^T as the epilogue of the second small product: one pass over the output
            # instead of three (product, scaling, sum)
            return _linear_plus_low_rank(self.linear, x, self.lora_dropout, self.lora_A, self.lora_B, self.scaling)
        return self.linear(x) + self.rms_norm(self._lora_branch(x))


def _linear_plus_low_rank(linear: nn.Linear, x: torch.Tensor, dropout, a: torch.Tensor, b: torch.Tensor, scaling: float) -> torch.Tensor:
    """``linear(x) + scaling · (dropout(x) a^T) b^T`` with the sum and the scaling in the epilogue of the second small
    product, written over the fresh output of the frozen linear (which nothing else holds and whose backward does not
    need it). Everything runs on the rows as a 2-d matrix and the result is viewed back: an in-place update through a
    view of a 3-d output would cost three copies of the output in the backward pass."""
    rows = x.reshape(-1, x.shape[-1])
    out = linear(rows)
    out.addmm_(F.linear(dropout(rows), a), b.t(), alpha=scaling)
    return out.view(*x.shape[:-1], out.shape[-1])


class LoRAQKVLinear(LoRALinear):
    """LoRA on the fused qkv projection, separately enabled for q, k and v."""

    def __init__(self, in_features: int, head_size: int, n_head: int, n_query_groups: int, r: int = 0, lora_alpha: int = 1,
                 lora_dropout: float = 0.0, enable_lora: Union[bool, Tuple[bool, bool, bool]] = False,
                 use_rms_norm: bool = False, **kwargs):
        nn.Module.__init__(self)
        self.r, self.lora_alpha = r, lora_alpha
        self.lora_dropout = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        self.merged = False
        out_features = head_size * (n_head + 2 * n_query_groups)
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        self.head_size, self.n_head, self.n_query_groups = head_size, n_head, n_query_groups
        if isinstance(enable_lora, bool):
            enable_lora = [enable_lora] * 3
        assert len(enable_lora) == 3
        self.enable_lora = list(enable_lora)
        self._all_qkv_shapes = (head_size * n_head, head_size * n_query_groups, head_size * n_query_groups)
        self.rms_norm = None
        if r > 0 and any(enable_lora):
            self.lora_A = nn.Parameter(torch.empty((r * sum(enable_lora), in_features)))
            self.qkv_shapes = [s for s, e in zip(self._all_qkv_shapes, enable_lora) if e]
            self.lora_B = nn.Parameter(torch.empty(sum(self.qkv_shapes), r))
            self.scaling = lora_alpha / r
            if use_rms_norm:
                self.rms_norm = RMSNorm(out_features)
            self.reset_parameters()

    def _parts(self):
        """(output offset, output size, A rows, B rows) of every enabled part."""
        out_off = a_off = b_off = 0
        for size, enabled in zip(self._all_qkv_shapes, self.enable_lora):
            if enabled:
                yield out_off, size, slice(a_off, a_off + self.r), slice(b_off, b_off + size)
                a_off += self.r
                b_off += size
            out_off += size

    def zero_pad(self, x: torch.Tensor) -> torch.Tensor:
        """Scatter the enabled parts ``(..., Σ enabled)`` into ``(..., out_features)``."""
        if all(self.enable_lora):
            return x
        result = x.new_zeros(*x.shape[:-1], self.linear.out_features)
        off = 0
        for out_off, size, _, _ in self._parts():
            result[..., out_off : out_off + size] = x[..., off : off + size]
            off += size
        return result

    def get_lora_AB(self) -> torch.Tensor:
        delta = self.lora_A.new_zeros(self.linear.out_features, self.linear.in_features)
        for out_off, size, a_rows, b_rows in self._parts():
            delta[out_off : out_off + size] = self.lora_B[b_rows] @ self.lora_A[a_rows]
        return delta * self.scaling

    def _lora_branch(self, x: torch.Tensor) -> torch.Tensor:
        after_a = F.linear(self.lora_dropout(x), self.lora_A)  # (..., r * n_enabled)
        pieces = [F.linear(after_a[..., a_rows], self.lora_B[b_rows]) for _, _, a_rows, b_rows in self._parts()]
        return self.zero_pad(torch.cat(pieces, dim=-1)) * self.scaling

    def _b_blocks(self) -> torch.Tensor:
        """``(out_features, r · n_enabled)``: B of every enabled part on its output rows and its rank columns, zeros
        elsewhere, so that one product serves all parts (and leaves the outputs of disabled parts alone)."""
        parts = list(self._parts())
        if len(parts) == 1 and parts[0][1] == self.linear.out_features:
            return self.lora_B
        blocks = self.lora_B.new_zeros(self.linear.out_features, self.lora_A.shape[0])
        for out_off, size, a_rows, b_rows in parts:
            blocks[out_off : out_off + size, a_rows] = self.lora_B[b_rows]
        return blocks

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.r == 0 or not any(self.enable_lora) or self.merged:
            return self.linear(x)
        if self.rms_norm is None:
            return _linear_plus_low_rank(self.linear, x, self.lora_dropout, self.lora_A, self._b_blocks(), self.scaling)
        return self.linear(x) + self.rms_norm(self._lora_branch(x))


# ---------------------------------------------------------------------- DoRA
def dora_forward(x, linear: nn.Linear, lora_ab: Optional[torch.Tensor], scales, eps: float) -> torch.Tensor:
    if lora_ab is None:
        return linear(x)
    merged = lora_ab + linear.weight.data
    norm = row_lengths(merged.detach(), eps)
    mult = (scales / norm).unsqueeze(-1).to(dtype=merged.dtype)
    return F.linear(x, merged * mult, linear.bias)


def dora_merge(linear: nn.Linear, lora_ab: torch.Tensor, scales, eps: float) -> None:
    dtype = linear.weight.data.dtype
    linear.weight.data += lora_ab.to(dtype)
    norm = row_lengths(linear.weight.data, eps)
    linear.weight.data *= (scales.data / norm).unsqueeze(-1).to(dtype=dtype)


class _DoRAMixin:
    _eps = 1e-9

    def _init_dora(self) -> None:
        has = hasattr(self, "lora_A")
        self.lora_scales = nn.Parameter(row_lengths(self.linear.weight.data, self._eps)) if has else None

    def reset_parameters(self) -> None:
        super().reset_parameters()
        if getattr(self, "lora_scales", None) is not None:
            self.lora_scales.data[:] = row_lengths(self.linear.weight.data, self._eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        do_lora = hasattr(self, "lora_A") and not self.merged
        return dora_forward(x, self.linear, self.get_lora_AB() if do_lora else None, self.lora_scales, self._eps)

    def merge(self) -> None:
        if hasattr(self, "lora_A") and not self.merged:
            dora_merge(self.linear, self.get_lora_AB(), self.lora_scales, self._eps)
            self.merged = True


class DoRALinear(_DoRAMixin, LoRALinear):
    def __init__(self, in_features, out_features, r=0, lora_alpha=1, eps: float = 1e-9, **kwargs):
        kwargs.pop("lora_dropout", None)
        kwargs.pop("use_rms_norm", None)
        self._eps = eps
        LoRALinear.__init__(self, in_features, out_features, r, lora_alpha, lora_dropout=0.0, **kwargs)
        self._init_dora()


class DoRAQKVLinear(_DoRAMixin, LoRAQKVLinear):
    def __init__(self, in_features, head_size, n_head, n_query_groups, r=0, lora_alpha=1, enable_lora=False, eps: float = 1e-9, **kwargs):
        kwargs.pop("lora_dropout", None)
        kwargs.pop("use_rms_norm", None)
        self._eps = eps
        LoRAQKVLinear.__init__(self, in_features, head_size, n_head, n_query_groups, r, lora_alpha, 0.0, enable_lora, **kwargs)
        self._init_dora()


def create_lora_linear(config: Config, in_size: int, out_size: int, bias: Optional[bool] = None, use_r: Optional[bool] = None):
    if bias is None:
        bias = config.bias
    if use_r is None:
        use_r = config.lora_mlp
    r = config.lora_r if use_r else 0
    if config.lora_kind == "dora":
        return DoRALinear(in_size, out_size, r=r, lora_alpha=config.lora_alpha, bias=bias)
    return LoRALinear(in_size, out_size, r=r, lora_alpha=config.lora_alpha, lora_dropout=config.lora_dropout,
                      use_rms_norm=config.lora_kind == "rms_norm", bias=bias)


def create_qkv_and_proj(config: Config):
    enable = (config.lora_query, config.lora_key, config.lora_value)
    common = dict(in_features=config.n_embd, head_size=config.head_size, n_head=config.n_head,
                  n_query_groups=config.n_query_groups, r=config.lora_r, lora_alpha=config.lora_alpha,
                  enable_lora=enable, bias=config.bias or config.attn_bias)
    if config.lora_kind == "dora":
        qkv = DoRAQKVLinear(**common)
    else:
        qkv = LoRAQKVLinear(**common, lora_dropout=config.lora_dropout, use_rms_norm=config.lora_kind == "rms_norm")
    proj = create_lora_linear(config, config.head_size * config.n_head, config.n_embd, use_r=config.lora_projection)
    return qkv, proj


def _remap(state_dict: Dict, prefix: str, names) -> None:
    """``<name>.weight`` → ``<name>.linear.weight`` for checkpoints of the base model."""
    for name in names:
        for attr in ("weight", "bias"):
            old, new = f"{prefix}{name}.{attr}", f"{prefix}{name}.linear.{attr}"
            if old in state_dict and new not in state_dict:
                state_dict[new] = state_dict.pop(old)


class CausalSelfAttention(base.CausalSelfAttention):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__(config, block_idx, kv_cache)
        self.qkv, self.proj = create_qkv_and_proj(config)

    def _load_from_state_dict(self, state_dict: Dict, prefix: str, *args: Any, **kwargs: Any) -> None:
        _remap(state_dict, prefix, ("qkv", "proj"))
        for attr in ("weight", "bias"):
            legacy = f"{prefix}attn.{attr}"
            if legacy in state_dict:
                state_dict[f"{prefix}qkv.linear.{attr}"] = base.qkv_reassemble(state_dict.pop(legacy), self.config)
        nn.Module._load_from_state_dict(self, state_dict, prefix, *args, **kwargs)


class GptNeoxMLP(base.GptNeoxMLP):
    def __init__(self, config: Config, intermediate_size: Optional[int] = None) -> None:
        super().__init__(config, intermediate_size)
        self.fc = create_lora_linear(config, config.n_embd, self.intermediate_size)
        self.proj = create_lora_linear(config, self.intermediate_size, config.n_embd)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        _remap(state_dict, prefix, ("fc", "proj"))
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class LLaMAMLP(base.LLaMAMLP):
    def __init__(self, config: Config, intermediate_size: Optional[int] = None) -> None:
        super().__init__(config, intermediate_size)
        self.fc_1 = create_lora_linear(config, config.n_embd, self.intermediate_size)
        self.fc_2 = create_lora_linear(config, config.n_embd, self.intermediate_size)
        self.proj = create_lora_linear(config, self.intermediate_size, config.n_embd)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        _remap(state_dict, prefix, ("fc_1", "fc_2", "proj"))
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class GemmaMLP(LLaMAMLP):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.gelu(self.fc_1(x), approximate=self.config.gelu_approximate) * self.fc_2(x))


class LLaMAMoE(base.LLaMAMoE):
    def __init__(self, config: Config) -> None:
        nn.Module.__init__(self)
        self.gate = create_lora_linear(config, config.n_embd, config.n_expert, bias=False)
        self.experts = nn.ModuleList(LLaMAMLP(config, intermediate_size=config.moe_intermediate_size) for _ in range(config.n_expert))
        self.config = config

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        _remap(state_dict, prefix, ("gate",))
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class Block(base.Block):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__(config, block_idx, kv_cache)
        self.attn = CausalSelfAttention(config, block_idx, kv_cache=kv_cache)
        self.mlp = config.mlp_class(config)


class GPT(base.GPT):
    def __init__(self, config: Config, **mha_kwargs) -> None:
        super().__init__(config, **mha_kwargs)
        self.lm_head = create_lora_linear(config, config.n_embd, config.padded_vocab_size, bias=config.lm_head_bias, use_r=config.lora_head)

    def _make_block(self, config, block_idx):
        return Block(config, block_idx)

    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "GPT":
        return cls(Config.from_name(name, **kwargs))

    def _init_weights(self, module: nn.Module) -> None:
        super()._init_weights(module)
        if isinstance(module, LoRALinear):
            module.reset_parameters()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        _remap(state_dict, prefix, ("lm_head",))
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


def mark_only_lora_as_trainable(model: nn.Module) -> None:
    """Freeze everything except the LoRA parameters (``lora_*``)."""
    for n, p in model.named_parameters():
        p.requires_grad = "lora_" in n or ".rms_norm." in n


def lora_filter(key: str, value: Any) -> bool:
    return "lora_" in key or ".rms_norm." in key


def merge_lora_weights(model: nn.Module) -> None:
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.merge()
