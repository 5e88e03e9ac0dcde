"""Single-token decode steps replayed from one CUDA graph.

A decode step of a 32-layer model is some six hundred small launches (five GEMMs, the norms, the
cache write, the split-KV attention, the score update and slot selection per layer): the host needs
longer to issue them than the GPU to run them. Once every cache is full, nothing in such a step
depends on the host any more except the position of the token: the slot to overwrite comes from
the previous step's selection (a device buffer; H2O) or follows from the position (last-recent ring), all
shapes are constant. The position is therefore
kept in a device word (``ops.cuda.device_position``): the cache write, the score normalisation and
the RoPE row read it there, and the captured step increments it. One ``cudaGraphLaunch`` then
replaces the launches of a step.

The reference decodes with eager PyTorch calls, one ``model(x)`` per token
(``keys_values/generate/base.py:50-57``, ``:219-347``); this module is used by
:func:`keys_values_b200.generate.base.batched_generate_fn` when :meth:`DecodeGraph.why_not`
returns ``None`` and falls back to the same eager call otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from keys_values_b200.models.model import GPT


class DecodeGraph:
    """Owns the captured step of ``model`` for batches of ``batch_size`` rows.

    ``step(tokens (B,1) int64) -> logits (B,1,V)``: the returned tensor is overwritten by the
    next call. Host-side counters of the caches advance with every step, so eager calls may
    follow at any time; after ``model.reset()`` or a new prefill the object must be dropped."""

    def __init__(self, model: GPT, batch_size: int):
        self.model = model
        self.batch_size = batch_size
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.tokens: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self.word: Optional[torch.Tensor] = None
        self.steps = 0

    # ------------------------------------------------------------------ conditions
    @staticmethod
    def why_not(model: GPT) -> Optional[str]:
        """``None`` if the next single-token step of ``model`` can be captured, else the reason."""
        from keys_values_b200.kvcache.basics import LastRecentlyInsertedKVCache
        from keys_values_b200.kvcache.h2o import H2OKVCache

        if not torch.cuda.is_available() or model.lm_head.weight.device.type != "cuda":
            return "model is not on a GPU"
        if model.start_of_layer_hook is not None:
            return "a start-of-layer hook is set"
        if torch.is_grad_enabled():
            return "gradients are enabled"
        for cache in model.get_kv_caches():
            if type(cache) is LastRecentlyInsertedKVCache:
                # ring of the most recent tokens: the slot is a function of the position
                if cache.current_length != cache.cache_length:
                    return "a cache is not full yet (its length still changes from step to step)"
            elif isinstance(cache, H2OKVCache) and cache._plain() and cache.max_chunk_size is not None:
                if cache.current_length != cache.cache_length or cache._use_initial_rule or cache._next_positions is None:
                    return "a cache is not full yet (its length still changes from step to step)"
                if cache.grace_period != 0:
                    return "grace_period > 0 keeps a ring position on the host"
                if cache.debug_next_positions is not None:
                    return "replay logging or recording is switched on"
            else:
                return "only last-recent caches and the plain H2O family with max_chunk_size choose their slots on the device"
            if cache._do_replay_log or cache.attn_recorder is not None:
                return "replay logging or recording is switched on"
            if not cache.kv_buffers.supports_direct_decode() or getattr(cache.kv_buffers, "before_access", None) is not None:
                return "the cache buffers are not read in place by the decode kernel"
        c = model.config
        if c.head_size != 128 or c.n_head % c.n_query_groups != 0:
            return "the decode kernel needs head size 128"
        return None

    # --------------------------------------------------------------------- capture
    def _advance_host(self) -> None:
        for cache in self.model.get_kv_caches():
            cache.advance_host_counters()

    def _capture(self, tokens: torch.Tensor) -> None:
        from keys_values_b200.ops import cuda as cu

        model = self.model
        dev = tokens.device
        input_pos = model.get_kv_caches()[0].input_pos
        self.tokens = tokens.clone()
        self.word = torch.tensor([input_pos], dtype=torch.int32, device=dev)
        self.graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(dev)
        comm = getattr(model, "tp_comm", None)  # tensor-parallel shard: its all-reduce calls take their epochs from a device word
        try:
            with cu.device_position(self.word):
                with torch.cuda.graph(self.graph):
                    if comm is not None:
                        comm.begin_capture()
                    self.logits = model(self.tokens)
                    self.word.add_(1)  # a scalar operand: nothing outside the graph's own memory is read here
                    if comm is not None:
                        comm.end_capture()
        except BaseException:
            if comm is not None:
                comm._capturing = False  # a failed capture must not leave later eager calls on the graph's sites
            self.graph = None
            raise
        # Capturing ran the host side of one step (the caches' counters moved on) without running
        # its kernels: the first replay is that step.

    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        model = self.model
        input_pos = model.get_kv_caches()[0].input_pos
        if input_pos + 1 > model.max_seq_length:
            raise ValueError(f"Cannot forward sequence: input_pos {input_pos} + 1 > max_seq_length {model.max_seq_length}")
        if self.graph is None:
            self._capture(tokens)  # moves the host counters on, like every eager call
        else:
            self.tokens.copy_(tokens)
            self._advance_host()
        self.graph.replay()
        self.steps += 1
        return self.logits


class Decoder:
    """``decoder(tokens (B,1)) -> logits (B,1,V)``: eager ``model(x)`` until the step can be captured
    (``warmup`` eager single-token steps come first, so that libraries have their handles and
    work spaces), then graph replays. ``use_graph=False`` keeps it eager."""

    def __init__(self, model: GPT, batch_size: int, use_graph: bool = True, warmup: int = 2):
        self.model = model
        self.batch_size = batch_size
        self.use_graph = use_graph
        self.warmup = warmup
        self.eager_steps = 0
        self.graph: Optional[DecodeGraph] = None
        self.reason: Optional[str] = None

    def __call__(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.graph is not None:
            return self.graph.step(tokens)
        if self.use_graph and self.eager_steps >= self.warmup and tokens.shape == (self.batch_size, 1):
            self.reason = DecodeGraph.why_not(self.model)
            if self.reason is None:
                self.graph = DecodeGraph(self.model, self.batch_size)
                return self.graph.step(tokens)
        self.eager_steps += 1
        return self.model(tokens)
