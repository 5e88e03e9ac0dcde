"""Rotary position encodings (linear, Llama-3 "adjusted", dynamic YaRN).

Parity: ``keys_values/pos_encoding.py:112-414``. The cos/sin tables depend on
the current context width, and for YaRN so does the SDPA scale factor
(``scale = (0.1·ln(factor)+1)² / sqrt(D)``), which is why both are inputs of the
kernels rather than compile-time constants.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch

from keys_values_b200.config import Config
from keys_values_b200.ops import reference as ref


def _position_context():
    from keys_values_b200 import ops

    return ops.position_context()

DEFAULT_YARN_ALPHA = 1.0
DEFAULT_YARN_BETA = 32.0


def build_rope_cache(
    seq_len: int,
    n_elem: int,
    device: Optional[torch.device] = None,
    base: float = 10000,
    condense_ratio: int = 1,
    extra_config: Optional[dict] = None,
    rope_local_base_freq: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables of shape ``(seq_len, n_elem)`` (or ``(seq_len, n_elem, 2)``
    with a local base frequency: index 0 = global, 1 = local)."""
    theta = 1.0 / (base ** (torch.arange(0, n_elem, 2, device=device).float() / n_elem))
    if extra_config is not None:
        factor = extra_config["factor"]
        if "original_max_seq_len" in extra_config:
            orig = extra_config["original_max_seq_len"]
            low = extra_config["low_freq_factor"]
            high = extra_config["high_freq_factor"]
            wavelen = 2 * math.pi / theta
            ratio = orig / wavelen
            smooth = torch.clamp((ratio - low) / (high - low), min=0.0, max=1.0)
            theta = (1 - smooth) * (theta / factor) + smooth * theta
        else:
            theta = theta / factor
    seq_idx = torch.arange(seq_len, device=device).float() / condense_ratio
    idx_theta = torch.outer(seq_idx, theta).repeat(1, 2)
    if idx_theta.shape[-1] > n_elem > 1:
        idx_theta = idx_theta[..., :n_elem]
    if rope_local_base_freq is not None:
        local_theta = 1.0 / (rope_local_base_freq ** (torch.arange(0, n_elem, 2, device=device).float() / n_elem))
        local_idx = torch.outer(seq_idx, local_theta).repeat(1, 2)
        if local_idx.shape[-1] > n_elem > 1:
            local_idx = local_idx[..., :n_elem]
        idx_theta = torch.stack((idx_theta, local_idx), dim=-1)
    return torch.cos(idx_theta), torch.sin(idx_theta)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return ref.apply_rope(x, cos, sin)


class PositionEncoding:
    """Interface: encode ``x (..., T, n_elem)`` for positions ``input_pos …``."""

    def __call__(self, x: torch.Tensor, input_pos: int, block_idx: int, **kwargs) -> torch.Tensor:
        raise NotImplementedError

    def sdpa_scale_factor(self) -> float:
        raise NotImplementedError

    @property
    def context_width(self) -> int:
        raise NotImplementedError

    def set_context_width(self, width: int):
        raise NotImplementedError

    def tables(self, input_pos: int, length: int, block_idx: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError


class LinearPositionEncoding(PositionEncoding):
    """Linear interpolation with a fixed factor (``config.rope_adjustments['factor']``)
    and fixed attention scale; supports Gemma-3 style local/global bases."""

    def __init__(self, config: Config, device: Optional[torch.device] = None, do_set_context_width: bool = True):
        self.rope_base = config.rope_base
        self.n_elem = config.rope_n_elem
        self.condense_ratio = config.rope_condense_ratio
        self.rope_local_base_freq = config.rope_local_base_freq
        self.rope_indices = config.rope_indices
        self._fixed_factor = None
        if config.rope_adjustments is not None:
            self._fixed_factor = config.rope_adjustments.get("factor")
            if self._fixed_factor is None:
                raise ValueError("config.rope_adjustments must include 'factor'")
        self.train_context_width = config.block_size
        self._device = device if device is not None else torch.get_default_device()
        self._cos = self._sin = None
        temp = config.attention_scores_scalar if config.attention_scores_scalar is not None else config.head_size
        self._sdpa_scale_factor = 1.0 / math.sqrt(temp)
        self._context_width = config.block_size
        if do_set_context_width:
            self.set_context_width(self._context_width)

    @property
    def context_width(self) -> int:
        return self._context_width

    @property
    def device(self):
        return self._device

    def set_context_width(self, width: int):
        if width <= 0:
            raise ValueError(f"width = {width}: Must be positive")
        if width == self._context_width and self._cos is not None and not self._is_dynamic():
            return
        self._context_width = width
        self._precompute()

    def _is_dynamic(self) -> bool:
        return False

    def sdpa_scale_factor(self) -> float:
        return self._sdpa_scale_factor

    def _factor(self) -> float:
        if self._fixed_factor is None:
            return max(1.0, self.context_width / self.train_context_width)
        return self._fixed_factor

    def _precompute_extra_args(self) -> Optional[Dict[str, Any]]:
        return {"factor": self._factor()}

    def _precompute(self):
        self._cos, self._sin = build_rope_cache(
            seq_len=self.context_width,
            n_elem=self.n_elem,
            device=self._device,
            base=self.rope_base,
            condense_ratio=self.condense_ratio,
            extra_config=self._precompute_extra_args(),
            rope_local_base_freq=self.rope_local_base_freq,
        )

    def tables(self, input_pos: int, length: int, block_idx: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Slices ``(length, n_elem)`` of the cos/sin tables for ``block_idx``."""
        if input_pos < 0 or input_pos + length > self.context_width:
            raise ValueError(
                f"input_pos = {input_pos}, length = {length}: need 0 <= input_pos, input_pos + length <= {self.context_width}"
            )
        if self._cos.device != torch.device(device):
            self._device = torch.device(device)
            self._cos = self._cos.to(self._device)
            self._sin = self._sin.to(self._device)
        ctx = _position_context() if length == 1 else None
        if ctx is not None:
            # captured decode step: the row is gathered by the device-resident position, once per step
            ind = None if self.rope_local_base_freq is None else self.rope_indices[block_idx]
            key = ("rope", id(self), ind)
            rows = ctx.cache.get(key)
            if rows is None:
                cos, sin = (self._cos, self._sin) if ind is None else (self._cos[:, :, ind], self._sin[:, :, ind])
                rows = ctx.cache[key] = (cos.index_select(0, ctx.word), sin.index_select(0, ctx.word))
            return rows
        if self.rope_local_base_freq is None:
            return self._cos[input_pos : input_pos + length], self._sin[input_pos : input_pos + length]
        ind = self.rope_indices[block_idx]
        return self._cos[input_pos : input_pos + length, :, ind], self._sin[input_pos : input_pos + length, :, ind]

    def __call__(self, x: torch.Tensor, input_pos: int, block_idx: int, **kwargs) -> torch.Tensor:
        if x.ndim < 2 or x.shape[-1] != self.n_elem:
            raise ValueError(f"x.shape = {x.shape}, last dimension must be {self.n_elem}")
        cos, sin = self.tables(input_pos, x.shape[-2], block_idx, x.device)
        return apply_rope(x, cos.unsqueeze(0), sin.unsqueeze(0))


class AdjustedPositionEncoding(LinearPositionEncoding):
    """Non-dynamic Llama-3 style frequency adjustment (``rope_adjustments`` with
    ``factor, original_max_seq_len, low_freq_factor, high_freq_factor``)."""

    def __init__(self, config: Config, device: Optional[torch.device] = None):
        super().__init__(config, device, do_set_context_width=False)
        if config.rope_adjustments is None:
            raise ValueError("config.rope_adjustments must be given")
        self.train_context_width = config.rope_adjustments.get("original_max_seq_len")
        if self.train_context_width is None:
            raise ValueError("Must have config.rope_adjustments['original_max_seq_len']")
        alpha = config.rope_adjustments.get("low_freq_factor", DEFAULT_YARN_ALPHA)
        beta = config.rope_adjustments.get("high_freq_factor", DEFAULT_YARN_BETA)
        if not (0 < alpha < beta):
            raise ValueError(f"alpha = {alpha}, beta = {beta}: Must be 0 < alpha < beta")
        self.alpha, self.beta = alpha, beta
        self._context_width = None
        self.set_context_width(max(config.block_size, int(self._fixed_factor * self.train_context_width)))

    def _precompute_extra_args(self):
        return {
            **super()._precompute_extra_args(),
            "original_max_seq_len": self.train_context_width,
            "low_freq_factor": self.alpha,
            "high_freq_factor": self.beta,
        }


class YaRNPositionEncoding(LinearPositionEncoding):
    """Dynamic YaRN (Peng et al., ICLR 2024): the interpolation factor and the
    attention temperature follow the current context width."""

    def __init__(self, config: Config, alpha: Optional[float] = None, beta: Optional[float] = None, device=None):
        super().__init__(config, device, do_set_context_width=False)
        self.head_size = config.head_size
        train_context_width = None
        factor = None
        if config.rope_adjustments is not None:
            ra = config.rope_adjustments
            if ra.get("low_freq_factor") is not None:
                if alpha is not None and alpha != ra["low_freq_factor"]:
                    raise ValueError("Cannot have config.rope_adjustments['low_freq_factor'] and alpha")
                alpha = ra["low_freq_factor"]
            if ra.get("high_freq_factor") is not None:
                if beta is not None and beta != ra["high_freq_factor"]:
                    raise ValueError("Cannot have config.rope_adjustments['high_freq_factor'] and beta")
                beta = ra["high_freq_factor"]
            train_context_width = ra.get("original_max_seq_len")
            factor = ra.get("factor")
        if train_context_width is not None:
            self.train_context_width = train_context_width
        if factor is not None:
            self._context_width = int(factor * self.train_context_width)
        alpha = DEFAULT_YARN_ALPHA if alpha is None else alpha
        beta = DEFAULT_YARN_BETA if beta is None else beta
        if not (0 < alpha < beta):
            raise ValueError(f"alpha = {alpha}, beta = {beta}: Must be 0 < alpha < beta")
        self.alpha, self.beta = alpha, beta
        self._sdpa_scale_factor = None
        self._fixed_factor = None
        width = self._context_width
        self._context_width = None
        self.set_context_width(width)

    def _is_dynamic(self) -> bool:
        return True

    def _precompute_extra_args(self):
        return {
            "factor": self._factor(),
            "original_max_seq_len": self.train_context_width,
            "low_freq_factor": self.alpha,
            "high_freq_factor": self.beta,
        }

    def _precompute(self):
        super()._precompute()
        sqrt_inv_t = 0.1 * math.log(self._factor()) + 1.0
        self._sdpa_scale_factor = sqrt_inv_t * sqrt_inv_t / math.sqrt(self.head_size)


def position_encoding_factory(config: Config, do_yarn: bool = False, **kwargs) -> PositionEncoding:
    if do_yarn:
        return YaRNPositionEncoding(config, **kwargs)
    ra = config.rope_adjustments
    if ra is not None and "original_max_seq_len" in ra:
        return AdjustedPositionEncoding(config, **kwargs)
    return LinearPositionEncoding(config, **kwargs)
