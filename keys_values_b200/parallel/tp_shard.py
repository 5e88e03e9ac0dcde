"""Which tensor of a model goes where under tensor parallelism: the configuration of one rank's shard, the split of
plain and LoRA state dicts over ranks, and its inverse. Pure functions of names and shapes (no communication), used
by :mod:`keys_values_b200.parallel.tp` and by the checkpoint readers / writers.

Layout: the fused ``qkv`` projection and the MLP up projections are column parallel (a rank holds the rows of its
query heads / KV heads / MLP columns, and the rows of their LoRA ``B``; LoRA ``A`` is replicated), the attention and
MLP output projections are row parallel (a rank holds their columns and the columns of their LoRA ``A``; LoRA ``B`` and
the bias are replicated, the bias kept by rank 0). Everything else (embedding, norms, head) is replicated.
"""
from __future__ import annotations

import torch


def local_config(config, world: int):
    """The configuration of one rank's shard: heads, KV heads and MLP width divided by ``world``."""
    import dataclasses

    H, G, I = config.n_head, config.n_query_groups, config.intermediate_size
    if G % world or I % world:
        raise ValueError(f"n_query_groups = {G} and intermediate_size = {I} must be divisible by the tensor-parallel size {world}")
    if config.norm_qk and config.norm_qk_type == "olmo2":
        raise NotImplementedError("a QK norm over all heads at once cannot be sharded over heads")
    if config.mlp_class_name == "LLaMAMoE":
        raise NotImplementedError("mixture-of-experts blocks are not sharded")
    return dataclasses.replace(config, n_head=H // world, n_query_groups=G // world, intermediate_size=I // world, head_size=config.head_size)  # keeps the class: LoRA fields survive


def _shard_rule(key: str, config):
    """How the tensor ``key`` of a whole model is split over ranks: ``(kind, axis)`` with kind in
    ``rep`` (replicated), ``rank0`` (kept by rank 0, zero elsewhere: biases of row-parallel linears),
    ``qkv`` (the q | k | v row segments, each split over KV groups), ``qkv_lora`` (the same for the rows of the
    enabled segments of a LoRA ``B``), ``heads`` (the H·D axis), ``inter`` (the MLP axis)."""
    leaf = key.rsplit(".", 1)[-1]
    weight_like = leaf in ("weight", "bias")
    if ".attn.qkv." in key:
        if leaf == "lora_A":
            return "rep", 0
        if leaf == "lora_B":
            return "qkv_lora", 0
        return ("qkv", 0) if weight_like else ("rep", 0)
    if ".attn.proj." in key:
        if leaf == "weight" or leaf == "lora_A":
            return "heads", 1
        return ("rank0", 0) if leaf == "bias" else ("rep", 0)
    if ".mlp.fc" in key:
        if leaf == "lora_A":
            return "rep", 0
        return ("inter", 0) if (weight_like or leaf == "lora_B") else ("rep", 0)
    if ".mlp.proj." in key:
        if leaf == "weight" or leaf == "lora_A":
            return "inter", 1
        return ("rank0", 0) if leaf == "bias" else ("rep", 0)
    return "rep", 0


def _qkv_segments(config, rows: int):
    """Row segments ``(start, rows_per_group)`` of a fused q | k | v tensor with ``rows`` rows: all three for the
    projection itself, only the LoRA-enabled ones for a LoRA ``B``."""
    H, G, D = config.n_head, config.n_query_groups, config.head_size
    full = [(H // G) * D, D, D]  # rows per KV group of the q, k and v segments
    if rows == (H + 2 * G) * D:
        per_group = full
    else:
        enabled = [getattr(config, f"lora_{n}", False) for n in ("query", "key", "value")]
        per_group = [w for w, e in zip(full, enabled) if e]
        if rows != sum(per_group) * G:
            raise ValueError(f"cannot interpret a fused qkv tensor with {rows} rows")
    segs, start = [], 0
    for w in per_group:
        segs.append((start, w))
        start += w * G
    return segs


def shard_state_dict(state_dict, config, world: int, rank: int):
    """State dict of the whole model (plain or LoRA) → state dict of the shard of ``rank`` (see
    :func:`local_config`). Column-parallel linears keep their rows and the rows of their LoRA ``B`` (``A`` is
    replicated), row-parallel linears their columns and the columns of their LoRA ``A`` (``B`` is replicated)."""
    G, I = config.n_query_groups, config.intermediate_size
    D, gs = config.head_size, config.n_head // config.n_query_groups
    g0, g1 = rank * (G // world), (rank + 1) * (G // world)
    i0, i1 = rank * (I // world), (rank + 1) * (I // world)
    out = {}
    for key, t in state_dict.items():
        kind, axis = _shard_rule(key, config)
        if kind == "rep":
            out[key] = t
        elif kind == "rank0":
            out[key] = t if rank == 0 else torch.zeros_like(t)
        elif kind in ("qkv", "qkv_lora"):
            out[key] = torch.cat([t[s + g0 * w : s + g1 * w] for s, w in _qkv_segments(config, t.shape[0])]).contiguous()
        elif kind == "heads":
            out[key] = t.narrow(axis, g0 * gs * D, (g1 - g0) * gs * D).contiguous()
        else:
            out[key] = t.narrow(axis, i0, i1 - i0).contiguous()
    return out


def unshard_state_dict(shards, config):
    """Inverse of :func:`shard_state_dict`: the state dicts of all ranks (in rank order) → the whole model's."""
    world = len(shards)
    G = config.n_query_groups
    out = {}
    for key, t0 in shards[0].items():
        kind, axis = _shard_rule(key, config)
        if kind in ("rep", "rank0"):
            out[key] = t0
        elif kind in ("qkv", "qkv_lora"):
            rows = t0.shape[0] * world
            parts = []
            for s, w in _qkv_segments(config, rows):
                local_start = s // world
                for sh in shards:
                    parts.append(sh[key][local_start : local_start + w * (G // world)])
            out[key] = torch.cat(parts).contiguous()
        else:
            out[key] = torch.cat([sh[key] for sh in shards], dim=axis).contiguous()
    return out
