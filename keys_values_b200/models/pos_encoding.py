"""Rotary position encodings (linear, Llama-3 "adjusted", dynamic YaRN).

Parity: ``keys_values/pos_encoding.py:112-414``. The cos/sin tables depend on
the current context width, and for YaRN so does the SDPA scale factor
(``scale = (0.1·ln(factor)+1)² / sqrt(D)``), which is why both are inputs of the
kernels rather than compile-time constants.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
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


@dataclass(frozen=True)
class _Stretch:
    """How the rotary frequencies are stretched for one context width. ``ramp`` is ``None`` for a
    uniform stretch by ``by``; otherwise ``(trained_width, low, high)`` of the wavelength ramp that
    leaves high frequencies alone and stretches low ones by ``by``."""

    by: float
    ramp: Optional[Tuple[int, float, float]] = None

    def as_rope_cache_args(self) -> Dict[str, Any]:
        args: Dict[str, Any] = {"factor": self.by}
        if self.ramp is not None:
            args.update(original_max_seq_len=self.ramp[0], low_freq_factor=self.ramp[1], high_freq_factor=self.ramp[2])
        return args


def _ramp_bounds(low: Optional[float], high: Optional[float]) -> Tuple[float, float]:
    low = DEFAULT_YARN_ALPHA if low is None else low
    high = DEFAULT_YARN_BETA if high is None else high
    if not 0 < low < high:
        raise ValueError(f"frequency ramp needs 0 < low_freq_factor < high_freq_factor, got {low} and {high}")
    return low, high


class _RotaryTables(PositionEncoding):
    """Table engine shared by the three rotary variants. A variant says, for a context width, how the
    frequencies are stretched (:meth:`_stretch_for`) and which attention temperature goes with it
    (:meth:`_scale_for`); this class owns the cos / sin tables for the current width, rebuilds them
    when the answer for a new width differs, hands out row slices (or, inside a captured decode step,
    the row selected by the device-resident position), and applies the rotation."""

    def __init__(self, config: Config, device: Optional[torch.device]):
        self.n_elem = config.rope_n_elem
        self.rope_indices = config.rope_indices
        self._bases = (config.rope_base, config.rope_local_base_freq)
        self._condense = config.rope_condense_ratio
        self._plain_scale = 1.0 / math.sqrt(config.attention_scores_scalar or config.head_size)
        self._where = torch.device(device) if device is not None else torch.get_default_device()
        self._width = 0
        self._built_for: Optional[Tuple[int, _Stretch]] = None
        self._table: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        self._scale = self._plain_scale

    # -- what a variant decides
    def _stretch_for(self, width: int) -> _Stretch:
        raise NotImplementedError

    def _scale_for(self, width: int) -> float:
        return self._plain_scale

    # -- interface
    @property
    def context_width(self) -> int:
        return self._width

    @property
    def device(self) -> torch.device:
        return self._where

    def sdpa_scale_factor(self) -> float:
        return self._scale

    def set_context_width(self, width: int):
        if width <= 0:
            raise ValueError(f"context width must be positive, got {width}")
        self._width = int(width)
        self._scale = self._scale_for(self._width)
        wanted = (self._width, self._stretch_for(self._width))
        if wanted != self._built_for:
            self._table = build_rope_cache(
                seq_len=self._width, n_elem=self.n_elem, device=self._where, base=self._bases[0], condense_ratio=self._condense,
                extra_config=wanted[1].as_rope_cache_args(), rope_local_base_freq=self._bases[1],
            )
            self._built_for = wanted

    def _layer_tables(self, block_idx: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        device = torch.device(device)
        if self._table[0].device != device:
            self._where = device
            self._table = (self._table[0].to(device), self._table[1].to(device))
        if self._bases[1] is None:
            return self._table
        which = self.rope_indices[block_idx]  # 0: global base, 1: local base
        return self._table[0][:, :, which], self._table[1][:, :, which]

    def tables(self, input_pos: int, length: int, block_idx: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Rows ``input_pos … input_pos + length`` of the cos / sin tables of layer ``block_idx``."""
        if not 0 <= input_pos <= self._width - length:
            raise ValueError(f"positions {input_pos} … {input_pos + length} lie outside the context width {self._width}")
        cos, sin = self._layer_tables(block_idx, device)
        ctx = _position_context() if length == 1 else None
        if ctx is None:
            return cos[input_pos : input_pos + length], sin[input_pos : input_pos + length]
        # captured decode step: the row follows the device-resident position; gathered once per step and layer kind
        key = ("rope", id(self), None if self._bases[1] is None else self.rope_indices[block_idx])
        if key not in ctx.cache:
            ctx.cache[key] = (cos.index_select(0, ctx.word), sin.index_select(0, ctx.word))
        return ctx.cache[key]

    def __call__(self, x: torch.Tensor, input_pos: int, block_idx: int, **kwargs) -> torch.Tensor:
        if x.ndim < 2 or x.shape[-1] != self.n_elem:
            raise ValueError(f"expected (..., T, {self.n_elem}), got {tuple(x.shape)}")
        cos, sin = self.tables(input_pos, x.shape[-2], block_idx, x.device)
        return apply_rope(x, cos[None], sin[None])


class LinearPositionEncoding(_RotaryTables):
    """Position interpolation: every frequency is divided by one factor. The factor is
    ``config.rope_adjustments['factor']`` when the config carries adjustments, else it follows the
    context width (``max(1, width / block_size)``). The attention scale is the plain ``1/sqrt(D)``.
    Gemma-3 style local / global bases are supported through ``rope_local_base_freq``."""

    def __init__(self, config: Config, device: Optional[torch.device] = None, do_set_context_width: bool = True):
        super().__init__(config, device)
        self.train_context_width = config.block_size
        self._pinned: Optional[float] = None
        if config.rope_adjustments is not None:
            if "factor" not in config.rope_adjustments or config.rope_adjustments["factor"] is None:
                raise ValueError("rope_adjustments without a 'factor' entry")
            self._pinned = float(config.rope_adjustments["factor"])
        if do_set_context_width:
            self.set_context_width(config.block_size)

    def _stretch_by(self, width: int) -> float:
        return self._pinned if self._pinned is not None else max(1.0, width / self.train_context_width)

    def _stretch_for(self, width: int) -> _Stretch:
        return _Stretch(self._stretch_by(width))


class AdjustedPositionEncoding(LinearPositionEncoding):
    """Llama-3 style adjustment with a fixed factor: ``rope_adjustments`` holds ``factor``,
    ``original_max_seq_len`` and optionally ``low_freq_factor`` / ``high_freq_factor``. Changing the
    context width only changes the table length, never the frequencies."""

    def __init__(self, config: Config, device: Optional[torch.device] = None):
        adj = config.rope_adjustments or {}
        if adj.get("original_max_seq_len") is None:
            raise ValueError("rope_adjustments['original_max_seq_len'] is required for the adjusted encoding")
        super().__init__(config, device, do_set_context_width=False)
        self.train_context_width = int(adj["original_max_seq_len"])
        self.alpha, self.beta = _ramp_bounds(adj.get("low_freq_factor"), adj.get("high_freq_factor"))
        self.set_context_width(max(config.block_size, int(self._pinned * self.train_context_width)))

    def _stretch_for(self, width: int) -> _Stretch:
        return _Stretch(self._pinned, (self.train_context_width, self.alpha, self.beta))


class YaRNPositionEncoding(LinearPositionEncoding):
    """Dynamic YaRN (Peng et al., ICLR 2024). With ``s = max(1, width / trained_width)`` for the current
    context width, low frequencies are stretched by ``s`` along the ``alpha … beta`` wavelength ramp and
    the attention scale becomes ``(0.1·ln s + 1)² / sqrt(D)``; both follow :meth:`set_context_width`.
    ``rope_adjustments`` may supply the ramp bounds, the trained width and (through ``factor``) the
    initial context width; ``alpha`` / ``beta`` arguments must then agree with it."""

    def __init__(self, config: Config, alpha: Optional[float] = None, beta: Optional[float] = None, device=None):
        adj = dict(config.rope_adjustments or {})
        for name, given in (("low_freq_factor", alpha), ("high_freq_factor", beta)):
            if adj.get(name) is not None and given is not None and given != adj[name]:
                raise ValueError(f"rope_adjustments[{name!r}] = {adj[name]} contradicts the argument {given}")
        initial_factor = adj.pop("factor", None)
        _RotaryTables.__init__(self, config, device)
        self._pinned = None
        self.head_size = config.head_size
        self.train_context_width = int(adj.get("original_max_seq_len") or config.block_size)
        low, high = adj.get("low_freq_factor"), adj.get("high_freq_factor")
        self.alpha, self.beta = _ramp_bounds(alpha if low is None else low, beta if high is None else high)
        start = config.block_size if initial_factor is None else int(initial_factor * self.train_context_width)
        self.set_context_width(start)

    def _stretch_for(self, width: int) -> _Stretch:
        return _Stretch(self._stretch_by(width), (self.train_context_width, self.alpha, self.beta))

    def _scale_for(self, width: int) -> float:
        root = 0.1 * math.log(self._stretch_by(width)) + 1.0
        return root * root / math.sqrt(self.head_size)


def position_encoding_factory(config: Config, do_yarn: bool = False, **kwargs) -> PositionEncoding:
    if do_yarn:
        return YaRNPositionEncoding(config, **kwargs)
    if (config.rope_adjustments or {}).get("original_max_seq_len") is not None:
        return AdjustedPositionEncoding(config, **kwargs)
    return LinearPositionEncoding(config, **kwargs)
