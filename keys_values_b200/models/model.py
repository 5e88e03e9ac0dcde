"""Decoder-only transformer with a per-layer KV-cache slot.

LitGPT-shaped module tree (``lm_head``, ``transformer.{wte,h,ln_f}``, fused
``attn.qkv`` with q|k|v concatenated, ``attn.proj``, ``mlp.{fc_1,fc_2,proj}``), so
that ``lit_model.pth`` state dicts load unchanged. Parity:
``keys_values/model.py:50-881``.

One structural difference from the reference: a block can be applied to a
*cell* (several consecutive chunks) at once. Norms, QKV/MLP GEMMs and RoPE then
run once over all tokens of the cell, and only the cache update + SDPA runs
chunk by chunk (``chunk_sizes`` argument), because only that part carries a
dependency from one chunk to the next.
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from keys_values_b200 import ops
from keys_values_b200.attention.base import DefaultKeysAndValues, MultiHeadSelfAttention, do_softcapping
from keys_values_b200.config import Config


class RMSNorm(nn.Module):
    """Root-mean-square layer norm (``keys_values/model.py:855-881``)."""

    def __init__(self, size: int, dim: int = -1, eps: float = 1e-6, add_unit_offset: bool = False) -> None:
        super().__init__()
        assert dim == -1
        self.weight = nn.Parameter(torch.ones(size))
        self.eps = eps
        self.dim = dim
        self.add_unit_offset = add_unit_offset

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.add_unit_offset)

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor):
        """``(norm(x + residual), x + residual)`` in one pass over the data."""
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, self.add_unit_offset)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


class GptNeoxMLP(nn.Module):
    def __init__(self, config: Config, intermediate_size: Optional[int] = None) -> None:
        super().__init__()
        self.intermediate_size = intermediate_size or config.intermediate_size
        self.fc = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.proj = nn.Linear(self.intermediate_size, config.n_embd, bias=config.bias)
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.gelu(self.fc(x), approximate=self.config.gelu_approximate))


class LLaMAMLP(nn.Module):
    def __init__(self, config: Config, intermediate_size: Optional[int] = None) -> None:
        super().__init__()
        self.intermediate_size = intermediate_size or config.intermediate_size
        self.fc_1 = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.fc_2 = nn.Linear(config.n_embd, self.intermediate_size, bias=config.bias)
        self.proj = nn.Linear(self.intermediate_size, config.n_embd, bias=config.bias)
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(ops.swiglu(self.fc_1(x), self.fc_2(x)))


class GemmaMLP(LLaMAMLP):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.gelu(self.fc_1(x), approximate=self.config.gelu_approximate) * self.fc_2(x))


class LLaMAMoE(nn.Module):
    """Mixture of SwiGLU experts; all experts run locally."""

    def __init__(self, config: Config) -> None:
        super().__init__()
        self.gate = nn.Linear(config.n_embd, config.n_expert, bias=False)
        self.experts = nn.ModuleList(
            LLaMAMLP(config, intermediate_size=config.moe_intermediate_size) for _ in range(config.n_expert)
        )
        self.config = config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.size()
        x = x.view(-1, C)
        router = self.gate(x)
        probs, indices = torch.topk(router, self.config.n_expert_per_token)
        probs = probs.softmax(dim=1, dtype=torch.float).to(dtype=x.dtype)
        y = torch.zeros_like(x)
        for e, expert in enumerate(self.experts):
            token_idx, expert_idx = torch.where(indices == e)
            if token_idx.numel():
                y.index_add_(0, token_idx, probs[token_idx, expert_idx, None] * expert(x[token_idx]))
        return y.view(B, T, C)


def _chunk_bounds(total: int, chunk_sizes: Optional[Sequence[int]]):
    if not chunk_sizes:
        return [(0, total)]
    assert sum(chunk_sizes) == total, (chunk_sizes, total)
    bounds, s = [], 0
    for c in chunk_sizes:
        bounds.append((s, s + c))
        s += c
    return bounds


class CausalSelfAttention(nn.Module):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__()
        self.qkv = nn.Linear(
            config.n_embd, (config.n_head + 2 * config.n_query_groups) * config.head_size, bias=config.bias or config.attn_bias
        )
        self.proj = nn.Linear(config.head_size * config.n_head, config.n_embd, bias=config.bias)
        self.kv_cache = kv_cache
        if config.norm_qk:
            olmo = config.norm_qk_type == "olmo2"
            self.norm_q = config.norm_class(config.n_head * config.head_size if olmo else config.head_size, eps=config.norm_eps)
            self.norm_k = config.norm_class(
                config.n_query_groups * config.head_size if olmo else config.head_size, eps=config.norm_eps
            )
        else:
            self.norm_q = self.norm_k = None
        self.config = config
        self.block_idx = block_idx

    def _qkv_apply(self, x: torch.Tensor) -> torch.Tensor:
        return self.qkv(x)

    def _split_norm_rope(self, qkv: torch.Tensor, mha: MultiHeadSelfAttention, input_pos: int):
        c = self.config
        H, G, D = c.n_head, c.n_query_groups, c.head_size
        B, T, _ = qkv.shape
        cos = sin = None
        if c.rope_n_elem > 0:
            cos, sin = mha.pos_encoding.tables(input_pos, T, self.block_idx, qkv.device)
        if c.norm_qk and c.norm_qk_type == "olmo2":
            q, k, v = qkv.split((H * D, G * D, G * D), dim=-1)
            qkv = torch.cat((self.norm_q(q), self.norm_k(k), v), dim=-1)
            qw = kw = None
        elif c.norm_qk:
            qw, kw = self.norm_q.weight, self.norm_k.weight
            if not isinstance(self.norm_q, RMSNorm):
                raise NotImplementedError("per-head QK norm needs RMSNorm")
        else:
            qw = kw = None
        unit = bool(getattr(self.norm_q, "add_unit_offset", False))
        return ops.qknorm_rope(qkv, H, G, D, cos, sin, qw, kw, c.norm_eps, c.rope_n_elem, unit)

    def forward(
        self,
        x: torch.Tensor,
        token_idx: torch.Tensor,
        mha: MultiHeadSelfAttention,
        chunk_sizes: Optional[Sequence[int]] = None,
    ) -> torch.Tensor:
        return self.proj(self.attend(self._qkv_apply(x), token_idx, mha, chunk_sizes))

    def attend(self, qkv: torch.Tensor, token_idx: torch.Tensor, mha: MultiHeadSelfAttention,
               chunk_sizes: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Everything between the QKV projection and the output projection: split, QK norm, RoPE, cache update
        and attention. ``qkv (B, T, (H + 2G)·D)`` → ``(B, T, H·D)``."""
        B, T, _ = qkv.shape
        input_pos = 0 if self.kv_cache is None else self.kv_cache.input_pos
        q, k, v = self._split_norm_rope(qkv, mha, input_pos)
        if self.kv_cache is None:
            y, _ = mha(query=q, k_and_v=DefaultKeysAndValues(k, v), block_idx=self.block_idx)
        else:
            bounds = _chunk_bounds(T, chunk_sizes)
            if len(bounds) == 1:
                y = self.kv_cache(query=q, key=k, value=v, token_idx=token_idx)
            else:
                # torch.split, not slices: the backward of a split is ONE concatenation of the chunk
                # gradients, whereas every slice would allocate, zero and accumulate a gradient of
                # the size of the whole cell
                sizes = [e - s for s, e in bounds]
                qs, ks, vs = (torch.split(t, sizes, dim=2) for t in (q, k, v))
                tis = torch.split(token_idx, sizes, dim=1)
                parts = [self.kv_cache(query=qc, key=kc, value=vc, token_idx=ti) for qc, kc, vc, ti in zip(qs, ks, vs, tis)]
                y = torch.cat(parts, dim=1)
        return y

    def create_default_kv_cache(self, batch_size: int, dtype=None, max_sequence_length: Optional[int] = None, device=None):
        from keys_values_b200.kvcache.basics import DenseKVCache

        if max_sequence_length is None:
            max_sequence_length = self.config.block_size
        self.kv_cache = DenseKVCache.from_config(
            config=self.config, max_batch_size=batch_size, cache_length=max_sequence_length,
            block_idx=self.block_idx, dtype=dtype, device=device,
        )

    def _load_from_state_dict(self, state_dict: dict, prefix: str, *args: Any, **kwargs: Any) -> None:
        # Legacy LitGPT checkpoints store an interleaved ``attn.attn.weight``.
        for attr in ("weight", "bias"):
            legacy_key = f"{prefix}attn.{attr}"
            if legacy_key in state_dict:
                state_dict[f"{prefix}qkv.{attr}"] = qkv_reassemble(state_dict.pop(legacy_key), self.config)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


def qkv_reassemble(param: torch.Tensor, config: Config) -> torch.Tensor:
    """Interleaved per-group ``[q…q k v]`` layout → concatenated ``q | k | v``."""
    q_per_kv = config.n_head // config.n_query_groups
    qs, ks, vs = [], [], []
    for chunk in torch.chunk(param, config.n_query_groups):
        split = torch.split(chunk, [config.head_size * q_per_kv, config.head_size, config.head_size])
        qs.append(split[0]); ks.append(split[1]); vs.append(split[2])
    return torch.cat((torch.cat(qs), torch.cat(ks), torch.cat(vs)))


class Block(nn.Module):
    def __init__(self, config: Config, block_idx: int, kv_cache=None) -> None:
        super().__init__()
        if not config.parallel_residual and config.shared_attention_norm:
            raise NotImplementedError("No checkpoint amongst the ones we support uses this configuration")
        self.norm_1 = nn.Identity() if not config.norm_1 else config.norm_class(config.n_embd, eps=config.norm_eps)
        self.attn = CausalSelfAttention(config, block_idx, kv_cache=kv_cache)
        self.post_attention_norm = (
            config.norm_class(config.n_embd, eps=config.norm_eps) if config.post_attention_norm else nn.Identity()
        )
        self.norm_2 = (
            nn.Identity()
            if not config.norm_2
            else (None if config.shared_attention_norm else config.norm_class(config.n_embd, eps=config.norm_eps))
        )
        self.mlp = config.mlp_class(config)
        self.post_mlp_norm = config.norm_class(config.n_embd, eps=config.norm_eps) if config.post_mlp_norm else nn.Identity()
        self.config = config

    def forward(
        self,
        x: torch.Tensor,
        token_idx: torch.Tensor,
        mha: MultiHeadSelfAttention,
        chunk_sizes: Optional[Sequence[int]] = None,
    ) -> torch.Tensor:
        """Non-parallel residual: ``x + attn(norm_1(x))`` then ``x + mlp(norm_2(x))``;
        parallel residual: ``x + attn(norm_1(x)) + mlp(norm_2(x))``."""
        x_normed = self.norm_1(x)
        attn_out = self.attn(x_normed, token_idx=token_idx, mha=mha, chunk_sizes=chunk_sizes)
        attn_out = self.post_attention_norm(attn_out)
        if self.config.parallel_residual:
            if not self.config.shared_attention_norm:
                x_normed = self.norm_2(x)
            x = attn_out + x
        elif isinstance(self.norm_2, RMSNorm):
            x_normed, x = self.norm_2.forward_add(attn_out, x)  # residual add fused into the norm
        else:
            x = attn_out + x
            x_normed = self.norm_2(x)
        return self.post_mlp_norm(self.mlp(x_normed)) + x


StartOfLayerHook = Callable[[torch.Tensor, int], None]


class GPT(nn.Module):
    def __init__(self, config: Config, **mha_kwargs) -> None:
        super().__init__()
        assert config.padded_vocab_size is not None
        self.config = config
        self.lm_head = nn.Linear(config.n_embd, config.padded_vocab_size, bias=config.lm_head_bias)
        self.transformer = nn.ModuleDict(
            dict(
                wte=nn.Embedding(config.padded_vocab_size, config.n_embd),
                h=nn.ModuleList(self._make_block(config, i) for i in range(config.n_layer)),
                ln_f=config.norm_class(config.n_embd, eps=config.norm_eps),
            )
        )
        self.mha = MultiHeadSelfAttention(config, **mha_kwargs)
        self._max_seq_length = config.block_size
        self._start_of_layer_hook: Optional[StartOfLayerHook] = None
        self._default_kv_cache = False

    def _make_block(self, config: Config, block_idx: int) -> Block:
        return Block(config, block_idx)

    # ------------------------------------------------------------ properties
    @property
    def max_seq_length(self) -> int:
        return self._max_seq_length

    @max_seq_length.setter
    def max_seq_length(self, value: int) -> None:
        """Sets the context width of the position encoding (for YaRN also the SDPA
        scale). Must not change in the middle of an inference run, since cached
        keys are already encoded."""
        if value <= 0:
            raise ValueError(f"value = {value}, must be positive")
        self._max_seq_length = value
        self.mha.set_seq_length(value)
        for kv_cache in self.get_kv_caches():
            if kv_cache is not None:
                kv_cache.set_seq_length(value)

    @property
    def start_of_layer_hook(self) -> Optional[StartOfLayerHook]:
        return self._start_of_layer_hook

    def set_start_of_layer_hook(self, hook: Optional[StartOfLayerHook]) -> None:
        """``hook(x, block_idx)`` is called with the input of every layer (and with
        ``block_idx == n_layer`` for the final output) in :meth:`forward`."""
        self._start_of_layer_hook = hook

    def reset_parameters(self) -> None:
        self.max_seq_length = self.config.block_size

    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, nn.Linear):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                torch.nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)

    # ---------------------------------------------------------------- caches
    def get_kv_caches(self) -> List[Any]:
        return [block.attn.kv_cache for block in self.transformer.h]

    def assign_kv_caches(self, kv_caches: Sequence[Any]) -> None:
        """Assign one cache per layer; shapes must match the model."""
        if len(kv_caches) != self.config.n_layer:
            raise ValueError(f"kv_caches must have one entry per layer ({self.config.n_layer})")
        for cache, block in zip(kv_caches, self.transformer.h):
            self._check_kv_cache(cache)
            block.attn.kv_cache = cache
        self._default_kv_cache = False

    def _check_kv_cache(self, cache) -> None:
        if cache is None:
            return
        if cache.n_query_groups != self.config.n_query_groups or cache.head_size != self.config.head_size:
            raise ValueError(
                f"cache has n_query_groups={cache.n_query_groups}, head_size={cache.head_size}; "
                f"model has {self.config.n_query_groups}, {self.config.head_size}"
            )

    def set_kv_caches(self, batch_size: int, dtype=None, max_seq_length: Optional[int] = None, device=None) -> None:
        """Create dense default caches for all layers."""
        if max_seq_length is None:
            max_seq_length = self.max_seq_length
        if device is None:
            device = self.lm_head.weight.device
        if dtype is None:
            dtype = self.lm_head.weight.dtype
        for block in self.transformer.h:
            block.attn.create_default_kv_cache(batch_size, dtype=dtype, max_sequence_length=max_seq_length, device=device)
        self._default_kv_cache = True

    def clear_kv_caches(self) -> None:
        for block in self.transformer.h:
            block.attn.kv_cache = None
        self._default_kv_cache = False

    def reset(self) -> None:
        """Prepare for a new sequence batch: caches forget their content."""
        for cache in self.get_kv_caches():
            if cache is not None:
                cache.reset()

    def get_kv_cache_params(self, block_idx: int):
        cache = self.transformer.h[block_idx].attn.kv_cache
        return None if cache is None else cache.get_params()

    def kv_cache_max_forward_length(self) -> Optional[int]:
        caches = self.get_kv_caches()
        if any(c is None for c in caches):
            return None
        return min(c.max_forward_length() for c in caches)

    def kv_cache_max_prefill_length(self) -> Optional[int]:
        caches = self.get_kv_caches()
        if any(c is None for c in caches):
            return None
        lens = [c.max_prefill_length for c in caches]
        return None if any(l is None for l in lens) else min(lens)

    # --------------------------------------------------------------- forward
    def embed(self, idx: torch.Tensor) -> torch.Tensor:
        x = self.transformer.wte(idx)
        if self.config.scale_embeddings:
            x = x * torch.tensor(self.config.n_embd**0.5, dtype=x.dtype)
        return x

    def head(self, x: torch.Tensor) -> torch.Tensor:
        """``ln_f`` + ``lm_head`` + final soft-capping, clipped to ``padded_vocab_size``."""
        x = self.transformer.ln_f(x)
        return do_softcapping(self.lm_head(x), self.config.final_logit_softcapping)

    def forward(self, idx: torch.Tensor, skip_lm_head: bool = False, chunk_sizes: Optional[Sequence[int]] = None) -> torch.Tensor:
        """``idx (B, T)`` token ids. With caches assigned, the first call after
        :meth:`reset` is the prefill, later calls continue the sequence; positions
        are tracked by the caches. Returns logits ``(B, T, padded_vocab)`` or, with
        ``skip_lm_head``, the final hidden states before ``ln_f``."""
        if idx.ndim == 1:
            idx = idx.unsqueeze(0)
        T = idx.size(1)
        caches = self.get_kv_caches()
        input_pos = caches[0].input_pos if caches[0] is not None else 0
        if input_pos + T > self.max_seq_length:
            raise ValueError(f"Cannot forward sequence: input_pos {input_pos} + {T} > max_seq_length {self.max_seq_length}")
        x = self.embed(idx)
        hook = self._start_of_layer_hook
        for block_idx, block in enumerate(self.transformer.h):
            if hook is not None:
                hook(x, block_idx)
            x = block(x, idx, self.mha, chunk_sizes=chunk_sizes)
        if hook is not None:
            hook(x, self.config.n_layer)
        if skip_lm_head:
            return x
        return self.head(x)

    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "GPT":
        return cls(Config.from_name(name, **kwargs))

    def clone(self, device: Optional[torch.device] = None) -> "GPT":
        """Copy of the model (weights copied, caches cloned) on ``device``."""
        import copy

        caches = self.get_kv_caches()
        self.clear_kv_caches()
        hook = self._start_of_layer_hook
        self._start_of_layer_hook = None
        try:
            model_copy = copy.deepcopy(self)
        finally:
            for cache, block in zip(caches, self.transformer.h):
                block.attn.kv_cache = cache
            self._start_of_layer_hook = hook
        if device is not None:
            model_copy = model_copy.to(device)
        model_copy.assign_kv_caches([None if c is None else c.clone(device=device) for c in caches])
        return model_copy
