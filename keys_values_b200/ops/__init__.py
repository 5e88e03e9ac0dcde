"""Hot ops of the framework.

Every op has exactly one GPU implementation, a hand-written sm_100a kernel in
``keys_values_b200/csrc`` reached through :mod:`keys_values_b200.ops.cuda`, and a
plain PyTorch restatement in :mod:`keys_values_b200.ops.reference` that serves
CPU tensors and is the oracle in the tests. If the native library cannot be loaded
on a machine with a GPU, the first call raises. A CUDA tensor whose shape or dtype a
kernel does not cover (for example a head size that has no instantiation, fp16
activations for the fused norms) is served by the PyTorch restatement on the GPU, and
the first such call of each op says so in a ``RuntimeWarning``; set
``KVB200_STRICT_NATIVE=1`` to turn that into an error.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from keys_values_b200.ops import reference as ref


def _cuda():
    from keys_values_b200.ops import cuda as _c

    return _c


_NOTICED = set()
_NATIVE_ATTENTION = True


def set_native_attention(enabled: bool) -> None:
    """``False`` sends every attention call (also on a GPU) to the blocked PyTorch restatement: the
    debugging switch behind ``--sdpa.use_eager_sdpa_always``."""
    global _NATIVE_ATTENTION
    _NATIVE_ATTENTION = bool(enabled)


def set_tmp_array_limit_gb(limit_gb: Optional[float]) -> None:
    """Upper bound for the score matrix that the PyTorch restatement of attention materialises at a time
    (it loops over blocks of query rows beyond it): ``--sdpa.tmp_array_limit_gb``."""
    ref.TMP_ARRAY_LIMIT_GB = float(limit_gb) if limit_gb else ref.DEFAULT_TMP_ARRAY_LIMIT_GB


def _restatement_on_gpu(op: str, why: str) -> None:
    """Called when a CUDA tensor is about to be served by the PyTorch restatement."""
    import os
    import warnings

    msg = f"keys_values_b200.ops.{op}: no native kernel for {why}; using the PyTorch restatement on the GPU"
    if os.environ.get("KVB200_STRICT_NATIVE", "0") == "1":
        raise RuntimeError(msg)
    if (op, why) not in _NOTICED:
        _NOTICED.add((op, why))
        warnings.warn(msg, RuntimeWarning, stacklevel=3)


def check_status(device) -> None:
    """Synchronising check of the device status word (no-op for CPU devices): raises
    :class:`keys_values_b200.ops.cuda.NativeError` if a kernel reported that it gave up on a wait or
    skipped a bad index since the last check. Call it where the host reads a result anyway."""
    device = torch.device(device)
    if device.type == "cuda":
        _cuda().check_status(device)


def native_launches() -> int:
    """Number of native kernel launches issued by this process so far."""
    from keys_values_b200.ops import cuda as _c

    return _c.launch_count()


# ----------------------------------------------------------------- RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, add_unit_offset):
        y, rstd = _cuda().rmsnorm_fwd(x, weight, eps, add_unit_offset)
        ctx.save_for_backward(x, weight, rstd)
        ctx.add_unit_offset = add_unit_offset
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, rstd = ctx.saved_tensors
        need_w = weight is not None and ctx.needs_input_grad[1]
        dx, dw = _cuda().rmsnorm_bwd(gy.contiguous(), x, weight, rstd, ctx.add_unit_offset, need_w)
        return dx, dw, None, None


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, add_unit_offset: bool = False) -> torch.Tensor:
    if x.is_cuda:
        return _RMSNormFn.apply(x.contiguous(), weight, eps, add_unit_offset)
    return ref.rmsnorm(x, weight, eps, add_unit_offset)


class _AddRMSNormFn(torch.autograd.Function):
    """``s = x + res; y = rmsnorm(s) · w`` in one pass; the backward pass adds the gradient that
    reaches ``s`` through its other consumer (the residual path) in the same kernel."""

    @staticmethod
    def forward(ctx, x, res, weight, eps, add_unit_offset):
        y, s, rstd = _cuda().add_rmsnorm_fwd(x, res, weight, eps, add_unit_offset)
        ctx.save_for_backward(s, weight, rstd)
        ctx.add_unit_offset = add_unit_offset
        return y, s

    @staticmethod
    def backward(ctx, gy, gs):
        s, weight, rstd = ctx.saved_tensors
        need_w = weight is not None and ctx.needs_input_grad[2]
        if need_w or gy is None:
            # trainable norm weights: the general kernel, then the add
            if gy is None:
                return gs, gs, None, None, None
            dx, dw = _cuda().rmsnorm_bwd(gy.contiguous(), s, weight, rstd, ctx.add_unit_offset, need_w)
            if gs is not None:
                dx = dx + gs
            return dx, dx, dw, None, None
        gadd = None if gs is None else gs.contiguous()
        dx = _cuda().rmsnorm_bwd_add(gy.contiguous(), s, weight, rstd, gadd, ctx.add_unit_offset)
        return dx, dx, None, None, None


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                add_unit_offset: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(rmsnorm(x + res), x + res)``. One kernel on a GPU for bf16 rows of a supported
    width, the two separate ops otherwise."""
    if x.is_cuda and x.shape == res.shape and _cuda().add_rmsnorm_supported(x):
        return _AddRMSNormFn.apply(x.contiguous(), res.contiguous(), weight, eps, add_unit_offset)
    s = x + res
    return rmsnorm(s, weight, eps, add_unit_offset), s


# ------------------------------------------------------- QK-norm + RoPE + split
class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, q_weight, k_weight, H, G, D, eps, rope_n_elem, add_unit_offset):
        q, k, v, rstd = _cuda().qknorm_rope_fwd(qkv, cos, sin, q_weight, k_weight, H, G, D, eps, rope_n_elem, add_unit_offset)
        ctx.save_for_backward(qkv, cos, sin, q_weight, k_weight, rstd)
        ctx.meta = (H, G, D, eps, rope_n_elem, add_unit_offset)
        return q, k, v

    @staticmethod
    def backward(ctx, gq, gk, gv):
        qkv, cos, sin, q_weight, k_weight, rstd = ctx.saved_tensors
        H, G, D, eps, rope_n_elem, add_unit_offset = ctx.meta
        need_w = q_weight is not None and (ctx.needs_input_grad[3] or ctx.needs_input_grad[4])
        dqkv, dqw, dkw = _cuda().qknorm_rope_bwd(
            gq.contiguous(), gk.contiguous(), gv.contiguous(), qkv, cos, sin, q_weight, k_weight, rstd,
            H, G, D, rope_n_elem, add_unit_offset, need_w,
        )
        return dqkv, None, None, dqw, dkw, None, None, None, None, None, None


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
    """Fused split of ``qkv (B,T,(H+2G)D)`` + per-head RMSNorm of q/k + RoPE, giving
    ``q (B,H,T,D)``, ``k, v (B,G,T,D)`` contiguous."""
    if qkv.is_cuda and _cuda().qknorm_rope_supported(qkv, head_size, rope_n_elem):
        return _QKNormRopeFn.apply(
            qkv.contiguous(), cos, sin, q_weight, k_weight, n_head, n_query_groups, head_size, eps, rope_n_elem, add_unit_offset
        )
    if qkv.is_cuda:
        _restatement_on_gpu("qknorm_rope", f"head size {head_size}, {rope_n_elem} rotary elements, dtype {qkv.dtype}")
    return ref.qknorm_rope(qkv, n_head, n_query_groups, head_size, cos, sin, q_weight, k_weight, eps, rope_n_elem, add_unit_offset)


# ------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _cuda().swiglu_fwd(a, b)

    @staticmethod
    def backward(ctx, gy):
        a, b = ctx.saved_tensors
        return _cuda().swiglu_bwd(gy.contiguous(), a, b)


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        return _SwiGLUFn.apply(a.contiguous(), b.contiguous())
    return ref.swiglu(a, b)


# ------------------------------------------------------------------ attention
def sdpa_fwd(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    scale: float,
    input_pos: int,
    token_pos: Optional[torch.Tensor] = None,
    return_weights: bool = False,
    sliding_window: Optional[int] = None,
    softcap: Optional[float] = None,
):
    """Returns ``(out (B,q,H·D), weights (B,G,kv) fp32 | None, lse (B,H,q) fp32)``."""
    if query.is_cuda and _NATIVE_ATTENTION and _cuda().sdpa_supported(query, key, sliding_window, softcap):
        return _cuda().sdpa_fwd(query, key, value, scale, input_pos, token_pos, return_weights, sliding_window, softcap)
    if query.is_cuda and _NATIVE_ATTENTION:
        _restatement_on_gpu("sdpa_fwd", _sdpa_shape_text(query, sliding_window, softcap))
    return ref.sdpa(query, key, value, scale, input_pos, token_pos, return_weights, sliding_window, softcap, return_lse=True)


def _sdpa_shape_text(query, sliding_window, softcap) -> str:
    return (f"head size {query.shape[-1]}, dtype {query.dtype}"
            + (", sliding window" if sliding_window is not None else "") + (", logit soft-capping" if softcap is not None else ""))


def sdpa_bwd(
    grad_out: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    scale: float,
    input_pos: int,
    token_pos: Optional[torch.Tensor] = None,
    sliding_window: Optional[int] = None,
    softcap: Optional[float] = None,
    dk_accum: Optional[torch.Tensor] = None,
    dv_accum: Optional[torch.Tensor] = None,
):
    """Returns ``dq (B,H,q,D)``, ``dk, dv (B,G,kv,D)`` (fp32 for dk/dv). With
    ``dk_accum/dv_accum`` (fp32, cache shaped) the K/V gradients are added into their
    first ``kv`` slots instead and ``None`` is returned for them."""
    if query.is_cuda and _NATIVE_ATTENTION and _cuda().sdpa_bwd_supported(query, key, sliding_window, softcap):
        return _cuda().sdpa_bwd(grad_out, query, key, value, out, lse, scale, input_pos, token_pos, dk_accum, dv_accum,
                                sliding_window, softcap)
    if query.is_cuda and _NATIVE_ATTENTION:
        _restatement_on_gpu("sdpa_bwd", _sdpa_shape_text(query, sliding_window, softcap))
    dq, dk, dv = ref.sdpa_backward(grad_out, query, key, value, scale, input_pos, token_pos, sliding_window, softcap)
    if dk_accum is not None:
        L = key.shape[2]
        dk_accum[:, :, :L] += dk
        dv_accum[:, :, :L] += dv
        return dq, None, None
    return dq, dk, dv


class SDPAFunction(torch.autograd.Function):
    """Differentiable SDPA (no cache) on top of :func:`sdpa_fwd` / :func:`sdpa_bwd`
    (role of ``keys_values/attention/sdpa_op.py:254-371``)."""

    @staticmethod
    def forward(ctx, query, key, value, scale, input_pos, token_pos, sliding_window, softcap):
        out, _, lse = sdpa_fwd(query, key, value, scale, input_pos, token_pos, False, sliding_window, softcap)
        ctx.save_for_backward(query, key, value, out, lse, token_pos)
        ctx.meta = (scale, input_pos, sliding_window, softcap)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, value, out, lse, token_pos = ctx.saved_tensors
        scale, input_pos, sliding_window, softcap = ctx.meta
        dq, dk, dv = sdpa_bwd(grad_out.contiguous(), query, key, value, out, lse, scale, input_pos, token_pos, sliding_window, softcap)
        return dq.to(query.dtype), dk.to(key.dtype), dv.to(value.dtype), None, None, None, None, None


def sdpa(query, key, value, scale, input_pos, token_pos=None, return_weights=False, sliding_window=None, softcap=None):
    """SDPA returning ``(out, weights)``; differentiable when weights are not requested."""
    if return_weights or not torch.is_grad_enabled() or not (query.requires_grad or key.requires_grad or value.requires_grad):
        out, w, _ = sdpa_fwd(query, key, value, scale, input_pos, token_pos, return_weights, sliding_window, softcap)
        return out, w
    return SDPAFunction.apply(query, key, value, scale, input_pos, token_pos, sliding_window, softcap), None


# ---------------------------------------------------------------- quantization
def quantize_rows(x: torch.Tensor, bits: int):
    if x.is_cuda:
        return _cuda().quantize_rows(x, bits)
    return ref.quantize_rows(x, bits)


def dequantize_rows(q: torch.Tensor, scale: torch.Tensor, zp: torch.Tensor, bits: int, dtype: torch.dtype, out: Optional[torch.Tensor] = None):
    if q.is_cuda:
        return _cuda().dequantize_rows(q, scale, zp, bits, dtype, out)
    res = ref.dequantize_rows(q, scale, zp, bits, dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


# ------------------------------------------------------------ cache primitives
def cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos: int) -> None:
    if k_buf.is_cuda:
        return _cuda().cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos)
    return ref.cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos)


def cache_write_quant(k_buf, v_buf, token_pos, slots, key, value, input_pos: int, qk, sk, zk, qv, sv, zv, bits: int) -> None:
    """:func:`cache_write` into the full-precision scratch ``k_buf/v_buf`` (skipped if
    ``None``) fused with quantize-on-write of the same rows into the quantized
    storage ``q* (B,G,C,D|D/2) uint8``, ``s* (B,G,C) fp32``, ``z* (B,G,C) int32``."""
    if key.is_cuda:
        return _cuda().cache_write_quant(k_buf, v_buf, token_pos, slots, key, value, input_pos, qk, sk, zk, qv, sv, zv, bits)
    B = key.shape[0]
    idx = slots.to(torch.int64)
    if k_buf is not None:
        ref.cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos)
    else:
        n = key.shape[2]
        pos = (input_pos + torch.arange(n, device=key.device, dtype=token_pos.dtype)).view(1, 1, n).expand(B, key.shape[1], n)
        token_pos[:B].scatter_(2, idx, pos)
    for x, q, s, z in ((key, qk, sk, zk), (value, qv, sv, zv)):
        xq, xs, xz = ref.quantize_rows(x, bits)
        q[:B].scatter_(2, idx.unsqueeze(-1).expand(-1, -1, -1, xq.shape[-1]), xq)
        s[:B].scatter_(2, idx, xs)
        z[:B].scatter_(2, idx, xz)


def h2o_update(scores, weights, k_select: int, n_evictable: int, normalize=False, token_pos=None, input_pos=0, prefill_length=0,
               out=None):
    """``weights=None`` selects without accumulating; ``out`` (int32 ``(B,G,k_select)``) receives the result."""
    if scores.is_cuda:
        return _cuda().h2o_update(scores, weights, k_select, n_evictable, normalize, token_pos, input_pos, prefill_length, out)
    res = ref.h2o_update(scores, weights, k_select, n_evictable, normalize, token_pos, input_pos, prefill_length)
    if out is not None:
        out.copy_(res)
        return out
    return res


def position_context():
    """The active device-resident position of a captured decode step (``ops.cuda.device_position``), or ``None``."""
    import sys

    mod = sys.modules.get("keys_values_b200.ops.cuda")
    return None if mod is None else mod.position_context()


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        loss, lse = _cuda().ce_loss_fwd(logits, targets, ignore_index)
        ctx.save_for_backward(logits, targets, lse)
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, g):
        logits, targets, lse = ctx.saved_tensors
        return _cuda().ce_loss_bwd(logits, targets, lse, g.float().contiguous(), ctx.ignore_index), None, None


def cross_entropy_rows(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Token cross-entropy per row of ``logits (N, V)`` (fp32 result, 0 for ignored targets). On a
    GPU the bf16 / fp32 logits are read in place (no fp32 copy) by the ``ce_loss`` kernels."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(-1) == 1:
        return _CrossEntropyFn.apply(logits, targets.reshape(-1).to(torch.int64).contiguous(), ignore_index)
    return torch.nn.functional.cross_entropy(logits.float(), targets.reshape(-1), ignore_index=ignore_index, reduction="none")


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Sum over positions of the token cross-entropy, per batch row: ``(B,)``."""
    B = logits.shape[0]
    return cross_entropy_rows(logits.reshape(-1, logits.shape[-1]), targets, ignore_index).view(B, -1).sum(dim=-1)


def decode_attention(query, key, value, scale, input_pos, token_pos=None, return_weights=False):
    """One new query token against ``key/value (B,G,L,D)`` (all slots hold tokens at or
    before the query position). Returns ``(out (B,1,H·D), weights (B,G,L) | None)``."""
    if query.is_cuda and _NATIVE_ATTENTION and _cuda().decode_supported(query, key.shape[1]):
        return _cuda().decode_attention(query, key.contiguous(), value.contiguous(), scale, key.shape[2], return_weights)
    if query.is_cuda and _NATIVE_ATTENTION:
        _restatement_on_gpu("decode_attention", f"head size {query.shape[-1]}, dtype {query.dtype}, {query.shape[1]} heads over {key.shape[1]} groups")
    out, w = ref.sdpa(query, key, value, scale, input_pos, token_pos, return_weights)
    return out, w


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """``logits (R, V)`` → int64 ``(R,)``: greedy sampling. On a GPU a two-stage kernel spreads the few rows of a
    decode step over the whole device."""
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and logits.ndim == 2 and logits.stride(-1) == 1 and logits.shape[0] <= 65535:
        return _cuda().argmax_rows(logits)
    return torch.argmax(logits, dim=-1)
