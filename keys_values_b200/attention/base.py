"""Multi-head self-attention front end.

Role of ``keys_values/attention/base.py:132-597``. The reference picks among seven
SDPA implementations and reorders/pads K and V because its fast backends cannot
mask on token positions. Here there is one implementation per device: the native
kernel masks on ``token_positions`` directly, so there is no reordering, no query
padding and no backend choice. The ``SDPA_IMPL_*`` names are kept so that calling
code can still pass them; they all select the same path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from keys_values_b200 import ops
from keys_values_b200.config import Config
from keys_values_b200.models.pos_encoding import PositionEncoding, position_encoding_factory

SDPA_IMPL_NATIVE = 0
SDPA_IMPL_PYTORCH = SDPA_IMPL_NATIVE
SDPA_IMPL_QPADDED_PYTORCH = SDPA_IMPL_NATIVE
SDPA_IMPL_EAGER_BLOCKS = SDPA_IMPL_NATIVE
SDPA_IMPL_EAGER_NO_BLOCKS = SDPA_IMPL_NATIVE
SDPA_IMPL_FLEXATTENTION = SDPA_IMPL_NATIVE
SDPA_IMPL_FLEXATT_WITH_WEIGHTS = SDPA_IMPL_NATIVE
SDPA_IMPL_FLASHINFER = SDPA_IMPL_NATIVE


class KeysAndValues:
    """Lazy access to the full K and V tensors of a cache
    (``keys_values/attention/base.py:46-93``)."""

    def keys(self) -> torch.Tensor:
        raise NotImplementedError

    def values(self) -> torch.Tensor:
        raise NotImplementedError

    def both(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.keys(), self.values()

    def clear(self):
        pass


class DefaultKeysAndValues(KeysAndValues):
    def __init__(self, keys: torch.Tensor, values: torch.Tensor):
        assert keys.ndim == 4 and values.ndim == 4 and keys.shape[:3] == values.shape[:3]
        self._keys, self._values = keys, values

    def keys(self) -> torch.Tensor:
        return self._keys

    def values(self) -> torch.Tensor:
        return self._values

    def clear(self):
        self._keys = self._values = None


def do_softcapping(x: torch.Tensor, thresh: Optional[float]) -> torch.Tensor:
    if thresh is not None:
        return torch.tanh(x / thresh) * thresh
    return x


class MultiHeadSelfAttention:
    """Maintains the position encoding and calls the SDPA op.

    ``__call__`` returns ``(attn_outputs (B, q, H·D), attn_weights (B, G, kv) | None)``.
    """

    def __init__(
        self,
        config: Config,
        pos_encoding: Optional[PositionEncoding] = None,
        mask_cache=None,
        sdpa_kernels=None,
        tmp_array_limit_gb=None,
        **_ignored,
    ) -> None:
        self.config = config
        self.pos_encoding = pos_encoding if pos_encoding is not None else position_encoding_factory(config)
        self.tmp_array_limit_gb = tmp_array_limit_gb

    def set_seq_length(self, value: int, device=None) -> None:
        self.pos_encoding.set_context_width(value)

    def sliding_window(self, block_idx: int) -> Optional[int]:
        c = self.config
        if c.sliding_window_size is not None and c.sliding_window_indices[block_idx] == 1:
            return c.sliding_window_size
        return None

    def __call__(
        self,
        query: torch.Tensor,
        k_and_v: KeysAndValues,
        block_idx: int,
        input_pos: Optional[int] = None,
        return_attn_weights: bool = False,
        token_positions: Optional[torch.Tensor] = None,
        return_lse: bool = False,
        **_kwargs,
    ):
        """With ``return_lse`` a third value is returned: the log-sum-exp ``(B, H, q)``
        fp32 of the attention rows (kept by the training forward pass so that the
        backward pass does not have to recompute the attention outputs)."""
        keys, values = k_and_v.both()
        q_len, kv_len = query.shape[2], keys.shape[2]
        if input_pos is None:
            input_pos = 0
        if token_positions is None and input_pos != kv_len - q_len:
            # Without token positions the keys are taken to be tokens 0 … kv_len-1
            input_pos = kv_len - q_len
        kwargs = dict(
            scale=self.pos_encoding.sdpa_scale_factor(),
            input_pos=input_pos,
            token_pos=token_positions,
            return_weights=return_attn_weights,
            sliding_window=self.sliding_window(block_idx),
            softcap=self.config.attention_logit_softcapping,
        )
        if return_lse:
            return ops.sdpa_fwd(query, keys, values, **kwargs)
        return ops.sdpa(query, keys, values, **kwargs)
