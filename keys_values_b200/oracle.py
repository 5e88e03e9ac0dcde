"""Independent oracle for losses and gradients through an evicting KV cache.

The chunked engine (:class:`keys_values_b200.kvcache.gradient.main.LongContextGradientModel`)
computes gradients cell by cell, with replayed eviction decisions, reversible buffer
updates and activation checkpoints. This module computes the same quantity in the most
direct way there is: ONE forward pass over the whole sequence with plain autograd, in
which the effect of every cache is expressed as an attention mask,

    token ``j`` is visible to the queries of chunk ``k``  iff  ``j`` is resident in the
    cache after chunk ``k`` has been written (and ``j`` is not in the future),

built from the replay log of an inference pass (which slot every token was written to).
Quantized buffers are expressed as values: a key / value row that a chunk reads from an
earlier cell has been through ``dq(q(x))`` (with a straight-through gradient), rows of the
same cell are exact, which is the rule of
:class:`keys_values_b200.kvcache.quant_buffers.QuantizedKVCacheBuffers`.

Nothing of the chunking, replay, checkpoint or kernel code is used here; the only shared
pieces are the stateless sub-modules of the model (norms, linears, RoPE tables). The role
is that of the whole-sequence comparisons in the reference's tests
(``test/kvcache/test_gradient.py:114``, ``test/kvcache/test_gradient_main.py:86``,
``test/attention/test_attn_weights.py:87-95``), extended to caches that evict.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from keys_values_b200.kvcache.base import KVCacheReplayLog


def visibility_from_replay_log(log: KVCacheReplayLog, batch_size: int, n_query_groups: int, device=None) -> torch.Tensor:
    """Boolean ``(B, G, T, T)``: entry ``[b, g, i, j]`` says whether the query at position ``i`` attends to
    token ``j`` in the cache whose insert decisions ``log`` records (no grace period)."""
    if log.grace_period:
        raise NotImplementedError("the oracle covers caches without a grace period")
    T = len(log)
    C = log.cache_length
    vis = torch.zeros((batch_size, n_query_groups, T, T), dtype=torch.bool, device=device)
    slot_token = torch.full((batch_size, n_query_groups, C), -1, dtype=torch.long, device=device)  # token held by each slot
    causal = torch.ones((T, T), dtype=torch.bool, device=device).tril()
    start = 0
    for num, slots in zip(log.token_chunks, log.slot_positions):
        new_tokens = torch.arange(start, start + num, device=device)
        if slots is None:
            # tokens fill the next free slots in order (prefill, or a cache that is not full yet)
            if start + num > C:
                raise ValueError("a chunk without recorded slots must fit into the free part of the cache")
            slot_token[:, :, start : start + num] = new_tokens
        else:
            slot_token.scatter_(2, slots.to(device=device, dtype=torch.long), new_tokens.expand(batch_size, n_query_groups, num))
        resident = torch.zeros((batch_size, n_query_groups, T), dtype=torch.bool, device=device)
        held = slot_token.clamp(min=0)
        resident.scatter_(2, held, slot_token >= 0)
        vis[:, :, start : start + num] = resident[:, :, None, :] & causal[start : start + num][None, None]
        start += num
    return vis


def quantize_dequantize(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Asymmetric affine quantization of every row (last axis) to ``bits`` bits and back:
    ``scale = max((max − min) / (2^bits − 1), eps)``, ``zp = −round(min / scale)``,
    ``q = clamp(round(x / scale) + zp, 0, 2^bits − 1)``, ``x̂ = (q − zp) · scale``."""
    xf = x.float()
    lo, hi = xf.amin(dim=-1, keepdim=True), xf.amax(dim=-1, keepdim=True)
    levels = float(2**bits - 1)
    scale = ((hi - lo) / levels).clamp(min=torch.finfo(torch.float32).eps)
    zp = -torch.round(lo / scale)
    q = (torch.round(xf / scale) + zp).clamp(0, levels)
    return ((q - zp) * scale).to(x.dtype)


@dataclass
class _LayerPlan:
    visible: torch.Tensor                 # (B, G, T, T) bool
    chunk_bounds: List[Tuple[int, int]]
    chunk_cell: List[int]                 # cell index of every chunk
    bits: Optional[int]                   # storage bits of quantized buffers, None for full precision


class _MaskedAttention(torch.nn.Module):
    """Stands in for a layer's cache during the oracle pass: attention of all queries against all
    keys of the sequence under the layer's visibility mask, in fp32 PyTorch ops."""

    def __init__(self, plan: _LayerPlan, scale: float, n_head: int):
        super().__init__()
        self.plan, self.scale, self.n_head = plan, scale, n_head
        self.input_pos = 0
        self.summed_weights: Optional[torch.Tensor] = None

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, token_idx: torch.Tensor) -> torch.Tensor:
        B, H, T, D = query.shape
        G = key.shape[1]
        rep = H // G
        plan = self.plan
        if plan.bits is not None:
            # straight-through: values change, gradients pass unchanged
            key_q = key + (quantize_dequantize(key, plan.bits) - key).detach()
            value_q = value + (quantize_dequantize(value, plan.bits) - value).detach()
        outs = []
        weights = torch.zeros((B, G, T), dtype=torch.float32, device=query.device)
        token_cell = torch.empty(T, dtype=torch.long, device=query.device)
        for (s, e), c in zip(plan.chunk_bounds, plan.chunk_cell):
            token_cell[s:e] = c
        for (s, e), c in zip(plan.chunk_bounds, plan.chunk_cell):
            k_eff, v_eff = key, value
            if plan.bits is not None:
                same_cell = (token_cell == c).view(1, 1, T, 1)
                k_eff = torch.where(same_cell, key, key_q)
                v_eff = torch.where(same_cell, value, value_q)
            q = query[:, :, s:e].float().view(B, G, rep, e - s, D)
            scores = torch.einsum("bgrqd,bgkd->bgrqk", q, k_eff.float()) * self.scale
            mask = plan.visible[:, :, s:e].unsqueeze(2)
            probs = torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)
            outs.append(torch.einsum("bgrqk,bgkd->bgrqd", probs, v_eff.float()).reshape(B, H, e - s, D))
            if s > 0:  # the prefill returns no weights
                weights = weights + probs.detach().sum(dim=(2, 3)) / rep
        self.summed_weights = weights
        y = torch.cat(outs, dim=2)
        return y.transpose(1, 2).reshape(B, T, H * D).to(query.dtype)


def _storage_bits(cache) -> Optional[int]:
    buffers = getattr(cache, "kv_buffers", None)
    quantizer = getattr(buffers, "quantizer_k", None)
    return None if quantizer is None else int(quantizer.num_bits)


def oracle_loss_and_gradients(
    gpt_model,
    head_model,
    input_ids: torch.Tensor,
    targets: torch.Tensor,
    replay_logs: Sequence[KVCacheReplayLog],
    cells: Optional[Sequence] = None,
    storage_bits: Optional[Sequence[Optional[int]]] = None,
) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Loss (mean over the batch of the per-row losses, each normalised by its number of targets) and the
    gradients of all trainable parameters of ``gpt_model`` / ``head_model``, for a sequence that was processed
    through caches whose insert decisions are ``replay_logs`` (one per layer). ``cells`` are the
    :class:`keys_values_b200.long_context.ChunksForCell` of the pass (needed for quantized buffers: rows are
    exact within a cell); ``storage_bits`` gives the bits per layer (default: read from the assigned caches)."""
    from keys_values_b200.long_context import compute_loss_for_chunk

    config = gpt_model.config
    B, T = input_ids.shape
    caches = gpt_model.get_kv_caches()
    if storage_bits is None:
        storage_bits = [_storage_bits(c) for c in caches]
    plans = []
    for layer, log in enumerate(replay_logs):
        if len(log) != T:
            raise ValueError(f"replay log of layer {layer} covers {len(log)} tokens, the sequence has {T}")
        bounds, s = [], 0
        for n in log.token_chunks:
            bounds.append((s, s + n))
            s += n
        chunk_cell = [0] * len(bounds)
        if cells is not None:
            for ci, cell in enumerate(cells):
                for k, (cs, ce) in enumerate(bounds):
                    if cell.start <= cs and ce <= cell.end:
                        chunk_cell[k] = ci
        plans.append(_LayerPlan(visibility_from_replay_log(log, B, config.n_query_groups, input_ids.device), bounds, chunk_cell,
                                storage_bits[layer]))
    blocks = list(gpt_model.transformer.h)
    params = [p for p in list(gpt_model.parameters()) + list(head_model.parameters()) if p.requires_grad]
    saved_grads = [p.grad for p in params]
    for p in params:
        p.grad = None
    stand_ins = []
    try:
        gpt_model.max_seq_length = T  # YaRN tables and attention scale follow the sequence length
        scale = gpt_model.mha.pos_encoding.sdpa_scale_factor()
        for block, plan in zip(blocks, plans):
            stand_ins.append(_MaskedAttention(plan, scale, config.n_head))
            block.attn.kv_cache = stand_ins[-1]
        x = gpt_model.embed(input_ids)
        for block in blocks:
            x = block(x, input_ids, gpt_model.mha, chunk_sizes=None)
        loss = compute_loss_for_chunk(gpt_model, head_model, x, targets, 0).float()
        num = head_model.num_target_entries(targets)
        if num is not None:
            loss = loss / num.clamp(min=1).to(loss.dtype)
        loss = loss.mean()
        loss.backward()
        names = {id(p): n for n, p in list(gpt_model.named_parameters()) + [("head." + n, p) for n, p in head_model.named_parameters()]}
        grads = {names[id(p)]: p.grad.detach().clone() for p in params if p.grad is not None}
    finally:
        for block, cache in zip(blocks, caches):
            block.attn.kv_cache = cache
        for p, g in zip(params, saved_grads):
            p.grad = g
    oracle_loss_and_gradients.last_summed_weights = [s.summed_weights for s in stand_ins]
    return loss.detach(), grads
