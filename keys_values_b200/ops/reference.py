"""Plain PyTorch restatements of every hot op.

These are the CPU path and the numerical oracle for the CUDA kernels: each CUDA
kernel in ``keys_values_b200/csrc`` is tested against the function of the same
name here, evaluated in fp32.

Semantics follow the reference library:
  * attention weights are summed over the query axis and *averaged* over the
    query heads of a KV group, fp32, shape ``(B, G, kv)``
    (``keys_values/attention/base.py:633-642``);
  * the causal mask is by token position, not by slot index
    (``keys_values/attention/attention_utils.py:205-260``);
  * quantization is asymmetric affine per row of ``D`` values
    (``keys_values/kvcache/quantize/pytorch.py:100-154``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

QUANT_EPS = torch.finfo(torch.float32).eps


# ---------------------------------------------------------------- normalisation
def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, add_unit_offset: bool = False) -> torch.Tensor:
    dtype = x.dtype
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1.0 + w) if add_unit_offset else y * w
    return y.to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x`` has shape ``(..., T, n_elem)``; ``cos``/``sin`` broadcast to it."""
    half = x.shape[-1] // 2
    xf = x.float()
    rotated = torch.cat((-xf[..., half:], xf[..., :half]), dim=-1)
    return (xf * cos.float() + rotated * sin.float()).to(x.dtype)


def qknorm_rope(
    qkv: torch.Tensor,
    n_head: int,
    n_query_groups: int,
    head_size: int,
    cos: Optional[torch.Tensor],
    sin: Optional[torch.Tensor],
    q_weight: Optional[torch.Tensor],
    k_weight: Optional[torch.Tensor],
    eps: float,
    rope_n_elem: int,
    add_unit_offset: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Split a fused ``qkv`` activation ``(B, T, (H+2G)·D)`` into ``q (B,H,T,D)``,
    ``k, v (B,G,T,D)``, apply per-head RMSNorm to q/k (if weights are given) and
    RoPE on the first ``rope_n_elem`` features (``keys_values/model.py:690-779``)."""
    B, T, _ = qkv.shape
    H, G, D = n_head, n_query_groups, head_size
    q, k, v = qkv.split((H * D, G * D, G * D), dim=-1)
    q = q.view(B, T, H, D).transpose(1, 2)
    k = k.view(B, T, G, D).transpose(1, 2)
    v = v.view(B, T, G, D).transpose(1, 2)
    if q_weight is not None:
        q = rmsnorm(q, q_weight, eps, add_unit_offset)
        k = rmsnorm(k, k_weight, eps, add_unit_offset)
    if rope_n_elem > 0 and cos is not None:
        c = cos.view(1, 1, T, -1)
        s = sin.view(1, 1, T, -1)
        if rope_n_elem == D:
            q = apply_rope(q, c, s)
            k = apply_rope(k, c, s)
        else:
            q = torch.cat((apply_rope(q[..., :rope_n_elem], c, s), q[..., rope_n_elem:]), dim=-1)
            k = torch.cat((apply_rope(k[..., :rope_n_elem], c, s), k[..., rope_n_elem:]), dim=-1)
    return q.contiguous(), k.contiguous(), v.contiguous()


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (torch.nn.functional.silu(a.float()) * b.float()).to(a.dtype)


# -------------------------------------------------------------------- attention
def build_mask(
    token_pos: Optional[torch.Tensor],
    input_pos: int,
    q_len: int,
    kv_len: int,
    batch: int,
    n_groups: int,
    device,
    sliding_window: Optional[int] = None,
) -> torch.Tensor:
    """Boolean mask ``(B, G, q, kv)``; ``True`` = may attend. Query ``i`` sits at
    absolute position ``input_pos + i``; slot ``j`` holds token
    ``token_pos[b, g, j]`` (``arange(kv)`` if ``token_pos`` is None)."""
    if token_pos is None:
        tp = torch.arange(kv_len, device=device, dtype=torch.int64).view(1, 1, 1, kv_len)
    else:
        tp = token_pos.to(torch.int64)
        if tp.ndim == 1:
            tp = tp.view(1, 1, kv_len)
        tp = tp.expand(batch, n_groups, kv_len).unsqueeze(2)
    qp = (input_pos + torch.arange(q_len, device=device, dtype=torch.int64)).view(1, 1, q_len, 1)
    mask = tp <= qp
    if sliding_window is not None:
        mask = mask & (tp > qp - sliding_window)
    return mask


DEFAULT_TMP_ARRAY_LIMIT_GB = 2.0
TMP_ARRAY_LIMIT_GB = DEFAULT_TMP_ARRAY_LIMIT_GB  # see keys_values_b200.ops.set_tmp_array_limit_gb


def sdpa(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    scale: float,
    input_pos: int,
    token_pos: Optional[torch.Tensor] = None,
    return_weights: bool = False,
    sliding_window: Optional[int] = None,
    softcap: Optional[float] = None,
    return_lse: bool = False,
):
    """Scaled dot product attention with a token-position causal mask.

    ``query (B,H,q,D)``, ``key/value (B,G,kv,D)``. Returns ``out (B,q,H·D)`` and,
    if requested, ``weights (B,G,kv)`` fp32 = softmax weights summed over the
    query axis and averaged over the ``H/G`` query heads of the group, and
    ``lse (B,H,q)`` fp32 (natural log). The fp32 score matrix is formed for blocks of query
    rows of at most ``TMP_ARRAY_LIMIT_GB`` at a time (role of the blocked eager SDPA of the
    reference, ``keys_values/attention/base.py:660-742``)."""
    B, H, q_len, D = query.shape
    G, kv_len = key.shape[1], key.shape[2]
    gs = H // G
    kf = key.float()
    vf = value.float()
    rows = max(1, int(TMP_ARRAY_LIMIT_GB * 2**30 / (4.0 * B * H * kv_len)))
    outs, lses = [], []
    weights = torch.zeros((B, G, kv_len), dtype=torch.float32, device=query.device) if return_weights else None
    for r0 in range(0, q_len, rows):
        r1 = min(q_len, r0 + rows)
        qf = query[:, :, r0:r1].float().reshape(B, G, gs, r1 - r0, D)
        scores = torch.einsum("bgsqd,bgkd->bgsqk", qf, kf) * scale
        if softcap is not None:
            scores = torch.tanh(scores / softcap) * softcap
        mask = build_mask(token_pos, input_pos + r0, r1 - r0, kv_len, B, G, query.device, sliding_window)
        scores = scores.masked_fill(~mask.unsqueeze(2), float("-inf"))
        lse = torch.logsumexp(scores, dim=-1)
        probs = torch.exp(scores - lse.unsqueeze(-1))
        outs.append(torch.einsum("bgsqk,bgkd->bgsqd", probs, vf).reshape(B, H, r1 - r0, D))
        lses.append(lse.reshape(B, H, r1 - r0))
        if return_weights:
            weights += probs.sum(dim=(2, 3)) / gs
    out = torch.cat(outs, dim=2).transpose(1, 2).reshape(B, q_len, H * D).to(query.dtype)
    if return_lse:
        return out, weights, torch.cat(lses, dim=2)
    return out, weights


def sdpa_backward(
    grad_out: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    scale: float,
    input_pos: int,
    token_pos: Optional[torch.Tensor] = None,
    sliding_window: Optional[int] = None,
    softcap: Optional[float] = None,
    head_block: int = 8,
):
    """Gradients of :func:`sdpa` w.r.t. ``query, key, value`` (fp32 math, looped over
    KV groups to bound the size of the score matrix). ``grad_out (B,q,H·D)``.
    Returns ``dq (B,H,q,D)``, ``dk, dv (B,G,kv,D)`` in fp32."""
    B, H, q_len, D = query.shape
    G, kv_len = key.shape[1], key.shape[2]
    gs = H // G
    go = grad_out.view(B, q_len, G, gs, D).permute(0, 2, 3, 1, 4).float()  # B,G,gs,q,D
    dq = torch.empty(B, G, gs, q_len, D, dtype=torch.float32, device=query.device)
    dk = torch.empty(B, G, kv_len, D, dtype=torch.float32, device=query.device)
    dv = torch.empty_like(dk)
    qv = query.view(B, G, gs, q_len, D)
    for g in range(G):
        tp = None if token_pos is None else (token_pos if token_pos.ndim == 1 else token_pos[:, g : g + 1])
        mask = build_mask(tp, input_pos, q_len, kv_len, B, 1, query.device, sliding_window)  # B,1,q,kv
        qf = qv[:, g].float()  # B,gs,q,D
        kf = key[:, g].float()  # B,kv,D
        vf = value[:, g].float()
        raw = torch.einsum("bsqd,bkd->bsqk", qf, kf) * scale
        if softcap is not None:
            t = torch.tanh(raw / softcap)
            s = t * softcap
        else:
            s = raw
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        g_o = go[:, g]  # B,gs,q,D
        dv[:, g] = torch.einsum("bsqk,bsqd->bkd", p, g_o)
        dp = torch.einsum("bsqd,bkd->bsqk", g_o, vf)
        ds = p * (dp - (dp * p).sum(dim=-1, keepdim=True))
        if softcap is not None:
            ds = ds * (1.0 - t * t)
        ds = ds * scale
        dq[:, g] = torch.einsum("bsqk,bkd->bsqd", ds, kf)
        dk[:, g] = torch.einsum("bsqk,bsqd->bkd", ds, qf)
    return dq.view(B, H, q_len, D), dk, dv


# ----------------------------------------------------------------- quantization
def quantize_rows(x: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Asymmetric affine quantization of each row (last axis, length ``D``).

    Returns ``q`` uint8 with last dim ``D`` (8 bit) or ``D/2`` (4 bit; element
    ``i`` in the high nibble, element ``i + D/2`` in the low nibble), ``scale``
    fp32 ``(...,)`` and ``zero_point`` int32 ``(...,)``."""
    assert bits in (4, 8)
    qmax = float(2**bits - 1)
    xf = x.float()
    mn = xf.amin(dim=-1)
    mx = xf.amax(dim=-1)
    scale = torch.clamp((mx - mn) / qmax, min=QUANT_EPS)
    zp = (0 - torch.round(mn / scale)).to(torch.int32)
    q = torch.clamp(torch.round(xf / scale.unsqueeze(-1)) + zp.unsqueeze(-1).float(), 0.0, qmax).to(torch.uint8)
    if bits == 4:
        half = x.shape[-1] // 2
        q = (q[..., :half] << 4) | q[..., half:]
    return q, scale, zp


def dequantize_rows(q: torch.Tensor, scale: torch.Tensor, zp: torch.Tensor, bits: int, dtype: torch.dtype) -> torch.Tensor:
    if bits == 4:
        q = torch.cat(((q >> 4) & 0xF, q & 0xF), dim=-1)
    return ((q.float() - zp.unsqueeze(-1).float()) * scale.unsqueeze(-1)).to(dtype)


# ------------------------------------------------------------- cache primitives
def cache_write(
    k_buf: torch.Tensor,
    v_buf: torch.Tensor,
    token_pos: torch.Tensor,
    slots: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    input_pos: int,
) -> None:
    """Scatter ``key/value (B,G,n,D)`` into ``k_buf/v_buf (B,G,C,D)`` at ``slots
    (B,G,n)`` and record ``token_pos[b,g,slot] = input_pos + i`` (in place)."""
    B, G, n, D = key.shape
    idx = slots.to(torch.int64)
    k_buf[:B].scatter_(2, idx.unsqueeze(-1).expand(-1, -1, -1, D), key.to(k_buf.dtype))
    v_buf[:B].scatter_(2, idx.unsqueeze(-1).expand(-1, -1, -1, D), value.to(v_buf.dtype))
    pos = (input_pos + torch.arange(n, device=key.device, dtype=token_pos.dtype)).view(1, 1, n).expand(B, G, n)
    token_pos[:B].scatter_(2, idx, pos)


def h2o_update(
    scores: torch.Tensor,
    weights: torch.Tensor,
    k_select: int,
    n_evictable: int,
    normalize: bool = False,
    token_pos: Optional[torch.Tensor] = None,
    input_pos: int = 0,
    prefill_length: int = 0,
) -> torch.Tensor:
    """``scores (B,G,C) += weights`` in place, then return the indices of the
    ``k_select`` smallest (optionally age-normalised) scores among the first
    ``n_evictable`` slots, ascending, int32 ``(B,G,k_select)``
    (``keys_values/kvcache/attn_weights.py:721-783``, ``h2o.py:175-199``)."""
    if weights is not None:  # None: selection only
        scores += weights
    s = scores[:, :, :n_evictable]
    if normalize:
        age = input_pos - torch.clamp(token_pos[:, :, :n_evictable].to(torch.int64), min=prefill_length - 1)
        s = s / age.clamp(min=1).to(s.dtype)
    _, idx = torch.topk(s, k=k_select, dim=-1, largest=False, sorted=True)
    return idx.to(torch.int32)


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Sum over positions of the token cross-entropy, per batch row: ``(B,)``."""
    B = logits.shape[0]
    loss = torch.nn.functional.cross_entropy(
        logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), ignore_index=ignore_index, reduction="none"
    )
    return loss.view(B, -1).sum(dim=-1)
