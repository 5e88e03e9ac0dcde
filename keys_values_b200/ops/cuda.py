"""ctypes bindings to ``libkvb200.so`` (the sm_100a kernels of ``keys_values_b200/csrc``).

The library is built in-tree by :mod:`keys_values_b200.build_ext` and loaded on
first use. Every wrapper allocates its outputs with torch, passes raw device
pointers plus the current CUDA stream, and checks the returned status code, so
a missing library or a rejected argument raises instead of silently running
something else. Kernels that contain device-side waits report through a status
word (see ``csrc/common.cuh``); :func:`check_status` reads it.
"""
from __future__ import annotations

import ctypes
import math
from pathlib import Path
from typing import Optional

import torch

_LIB = None
_LAUNCHES = 0
_STATUS = {}
_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = _ROOT / "libkvb200.so"

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_ERRORS = {
    -1: "invalid argument", -2: "misaligned pointer or stride", -3: "driver entry point unavailable",
    -4: "tensor map creation failed", -5: "kernel launch failed", -6: "unsupported configuration",
    -7: "problem too large for this kernel", -8: "CUDA runtime error",
}
_STATUS_TEXT = {
    1: "timeout waiting for a full (data ready) barrier", 2: "timeout waiting for an empty (slot free) barrier",
    3: "timeout waiting for an accumulator in tensor memory", 4: "timeout waiting for tensor memory to be released",
    5: "timeout waiting for a peer flag", 6: "timeout in an intra-CTA wait", 7: "slot index out of range",
}


class NativeError(RuntimeError):
    pass


def lib():
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise NativeError(
                f"{LIB_PATH} is missing: run `python -m keys_values_b200.build_ext` (CUDA tensors have no PyTorch fallback)"
            )
        _LIB = ctypes.CDLL(str(LIB_PATH))
        _LIB.kvb_sdpa_fwd_scratch_bytes.restype = ctypes.c_longlong
    return _LIB


def available() -> bool:
    return LIB_PATH.exists()


def launch_count() -> int:
    return _LAUNCHES


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise NativeError(f"{name}: {_ERRORS.get(rc, rc)}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ll(x) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(x))


def _code(dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise NativeError(f"dtype {dtype} is not supported by the native kernels")


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write their error code to."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device, clear: bool = True) -> None:
    """Synchronising read of the status word; raises if a kernel reported an error."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        if clear:
            w.zero_()
        raise NativeError(f"native kernel reported: {_STATUS_TEXT.get(code, code)}")


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


# ------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, add_unit_offset: bool):
    dim = x.shape[-1]
    rows = x.numel() // dim
    if weight is not None and weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib().kvb_rmsnorm_fwd(_p(x), _p(weight), _p(y), _p(rstd), _ll(rows), dim, ctypes.c_float(eps),
                                 int(add_unit_offset), _code(x.dtype), _stream(x)), "rmsnorm_fwd")
    _count()
    return y, rstd


# ----------------------------------------------------------- cross-entropy
def ce_loss_fwd(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int):
    """``logits (N, V)`` fp32 / bf16 with unit stride along V, ``targets (N,)`` int64. Returns the
    per-row loss and log-sum-exp, both fp32."""
    N, V = logits.shape
    loss = torch.empty(N, dtype=torch.float32, device=logits.device)
    lse = torch.empty(N, dtype=torch.float32, device=logits.device)
    _check(lib().kvb_ce_loss_fwd(_p(logits), _p(targets), _p(loss), _p(lse), _ll(N), V, _ll(logits.stride(0)), _ll(ignore_index),
                                 0 if logits.dtype == torch.float32 else 1, _stream(logits)), "ce_loss_fwd")
    _count()
    return loss, lse


_ARGMAX_SCRATCH: dict = {}


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Index of the largest entry of every row of ``logits (R, V)`` (fp32 / bf16, unit stride along V): int64 ``(R,)``."""
    R, V = logits.shape
    lib().kvb_argmax_scratch_bytes.restype = ctypes.c_longlong
    key = logits.device.index or 0
    buf = _ARGMAX_SCRATCH.get(key)
    need = int(lib().kvb_argmax_scratch_bytes(_ll(R)))
    if buf is None or buf.numel() < need:
        # counters first (zero between calls), partial results behind them: sized for at least 64 rows
        buf = _ARGMAX_SCRATCH[key] = torch.zeros(max(need, int(lib().kvb_argmax_scratch_bytes(_ll(64)))), dtype=torch.uint8, device=logits.device)
    out = torch.empty(R, dtype=torch.int64, device=logits.device)
    _check(lib().kvb_argmax_rows(_p(logits), _p(out), _p(buf), _ll(R), V, _ll(logits.stride(0)), 0 if logits.dtype == torch.float32 else 1,
                                 _stream(logits)), "argmax_rows")
    _count()
    return out


def ce_loss_bwd(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, grad: torch.Tensor, ignore_index: int):
    N, V = logits.shape
    dlogits = torch.empty((N, V), dtype=logits.dtype, device=logits.device)
    if logits.stride(0) != V:
        logits = logits.contiguous()
    _check(lib().kvb_ce_loss_bwd(_p(logits), _p(targets), _p(lse), _p(grad), _p(dlogits), _ll(N), V, _ll(V), _ll(ignore_index),
                                 0 if logits.dtype == torch.float32 else 1, _stream(logits)), "ce_loss_bwd")
    _count()
    return dlogits


_RMS_FAST_DIMS = (1024, 2048, 2560, 3072, 3584, 4096, 5120)


def add_rmsnorm_supported(x: torch.Tensor) -> bool:
    """Fused ``s = x + res; y = rmsnorm(s)`` (and its backward with a fused gradient add): bf16 rows
    that fit into the registers of a warp."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] in _RMS_FAST_DIMS and x.shape[-1] <= 3072


def add_rmsnorm_fwd(x: torch.Tensor, res: torch.Tensor, weight: Optional[torch.Tensor], eps: float, add_unit_offset: bool):
    dim = x.shape[-1]
    rows = x.numel() // dim
    if weight is not None and weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
    y, s = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib().kvb_add_rmsnorm_fwd(_p(x), _p(res), _p(weight), _p(y), _p(s), _p(rstd), _ll(rows), dim, ctypes.c_float(eps),
                                     int(add_unit_offset), _stream(x)), "add_rmsnorm_fwd")
    _count()
    return y, s, rstd


def rmsnorm_bwd_add(gy, x, weight, rstd, gadd, add_unit_offset: bool):
    """``rmsnorm_backward(gy) + gadd`` in one pass (no weight gradient)."""
    dim = x.shape[-1]
    rows = x.numel() // dim
    wt = None if weight is None else weight.to(x.dtype)
    dx = torch.empty_like(x)
    _check(lib().kvb_rmsnorm_bwd_add(_p(gy), _p(x), _p(wt), _p(rstd), _p(gadd), _p(dx), _ll(rows), dim, int(add_unit_offset),
                                     _stream(x)), "rmsnorm_bwd_add")
    _count()
    return dx


def rmsnorm_bwd(gy, x, weight, rstd, add_unit_offset: bool, need_w: bool):
    dim = x.shape[-1]
    rows = x.numel() // dim
    wt = None if weight is None else weight.to(x.dtype)
    dx = torch.empty_like(x)
    n_partial = min(296, (rows + 7) // 8)
    dw_partial = torch.empty((n_partial, dim), dtype=torch.float32, device=x.device) if need_w else None
    _check(lib().kvb_rmsnorm_bwd(_p(gy), _p(x), _p(wt), _p(rstd), _p(dx), _p(dw_partial), _ll(rows), dim,
                                 int(add_unit_offset), _code(x.dtype), n_partial, _stream(x)), "rmsnorm_bwd")
    _count()
    dw = dw_partial.sum(0).to(weight.dtype) if need_w else None
    return dx, dw


# --------------------------------------------------------- QK-norm + RoPE
def qknorm_rope_supported(qkv: torch.Tensor, head_size: int, rope_n_elem: int) -> bool:
    return qkv.dtype in _DTYPE_CODE and head_size <= 256 and rope_n_elem % 2 == 0


def qknorm_rope_fwd(qkv, cos, sin, q_weight, k_weight, H, G, D, eps, rope_n_elem, add_unit_offset):
    B, T, _ = qkv.shape
    dev, dt = qkv.device, qkv.dtype
    q = torch.empty((B, H, T, D), dtype=dt, device=dev)
    k = torch.empty((B, G, T, D), dtype=dt, device=dev)
    v = torch.empty((B, G, T, D), dtype=dt, device=dev)
    has_norm = q_weight is not None
    rstd = torch.empty((B, T, H + G), dtype=torch.float32, device=dev) if has_norm else None
    if rope_n_elem > 0 and cos is not None:
        cos_c = cos.float().contiguous()
        sin_c = sin.float().contiguous()
    else:
        cos_c = sin_c = None
        rope_n_elem = 0
    qw = None if q_weight is None else q_weight.to(dt)
    kw = None if k_weight is None else k_weight.to(dt)
    _check(lib().kvb_qknorm_rope_fwd(_p(qkv), _p(cos_c), _p(sin_c), _p(qw), _p(kw), _p(q), _p(k), _p(v), _p(rstd), B, T, H, G, D,
                                     ctypes.c_float(eps), rope_n_elem, int(add_unit_offset), _code(dt), _stream(qkv)),
           "qknorm_rope_fwd")
    _count()
    return q, k, v, rstd


def qknorm_rope_bwd(gq, gk, gv, qkv, cos, sin, q_weight, k_weight, rstd, H, G, D, rope_n_elem, add_unit_offset, need_w):
    B, T, _ = qkv.shape
    dt = qkv.dtype
    dqkv = torch.empty_like(qkv)
    if rope_n_elem > 0 and cos is not None:
        cos_c, sin_c = cos.float().contiguous(), sin.float().contiguous()
    else:
        cos_c = sin_c = None
        rope_n_elem = 0
    rows = B * T * (H + 2 * G)
    n_partial = min(296, (rows + 7) // 8)
    dw_partial = torch.empty((n_partial, 2, D), dtype=torch.float32, device=qkv.device) if need_w else None
    qw = None if q_weight is None else q_weight.to(dt)
    kw = None if k_weight is None else k_weight.to(dt)
    _check(lib().kvb_qknorm_rope_bwd(_p(gq), _p(gk), _p(gv), _p(qkv), _p(cos_c), _p(sin_c), _p(qw), _p(kw), _p(rstd), _p(dqkv),
                                     _p(dw_partial), B, T, H, G, D, rope_n_elem, int(add_unit_offset), _code(dt), n_partial,
                                     _stream(qkv)), "qknorm_rope_bwd")
    _count()
    if need_w:
        dw = dw_partial.sum(0)
        return dqkv, dw[0].to(q_weight.dtype), dw[1].to(k_weight.dtype)
    return dqkv, None, None


# ------------------------------------------------------------------ SwiGLU
def swiglu_fwd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    y = torch.empty_like(a)
    _check(lib().kvb_swiglu_fwd(_p(a), _p(b), _p(y), _ll(a.numel()), _code(a.dtype), _stream(a)), "swiglu_fwd")
    _count()
    return y


def swiglu_bwd(gy, a, b):
    da, db = torch.empty_like(a), torch.empty_like(b)
    _check(lib().kvb_swiglu_bwd(_p(gy), _p(a), _p(b), _p(da), _p(db), _ll(a.numel()), _code(a.dtype), _stream(a)), "swiglu_bwd")
    _count()
    return da, db


# ------------------------------------------------------------ quantization
def quantize_rows(x: torch.Tensor, bits: int):
    x = x.contiguous()
    D = x.shape[-1]
    rows = x.numel() // D
    q = torch.empty((*x.shape[:-1], D if bits == 8 else D // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    zp = torch.empty(x.shape[:-1], dtype=torch.int32, device=x.device)
    _check(lib().kvb_quantize_rows(_p(x), _p(q), _p(scale), _p(zp), _ll(rows), D, bits, _code(x.dtype), _stream(x)), "quantize_rows")
    _count()
    return q, scale, zp


def dequantize_rows(q, scale, zp, bits: int, dtype, out: Optional[torch.Tensor] = None):
    D = q.shape[-1] * (2 if bits == 4 else 1)
    lead = q.shape[:-1]
    if q.ndim != 4:
        q4 = q.reshape(1, 1, -1, q.shape[-1])
        s4, z4 = scale.reshape(1, 1, -1), zp.reshape(1, 1, -1)
    else:
        q4, s4, z4 = q, scale, zp
    if q4.stride(-1) != 1 or s4.stride(-1) != 1 or z4.stride() != s4.stride():
        q4, s4, z4 = q4.contiguous(), s4.contiguous(), z4.contiguous()
    B, G, n, _ = q4.shape
    if out is None:
        res = torch.empty((B, G, n, D), dtype=dtype, device=q.device)
    else:
        res = out.view(B, G, n, D) if out.ndim != 4 else out
        if res.stride(-1) != 1 or res.dtype != dtype:
            raise NativeError("dequantize_rows: out must have a contiguous last dimension and the requested dtype")
    _check(lib().kvb_dequantize_rows(_p(q4), _p(s4), _p(z4), _p(res), B, G, n, D, _ll(q4.stride(0)), _ll(q4.stride(1)),
                                     _ll(q4.stride(2)), _ll(s4.stride(0)), _ll(s4.stride(1)), _ll(res.stride(0)),
                                     _ll(res.stride(1)), _ll(res.stride(2)), bits, _code(dtype), _stream(q)), "dequantize_rows")
    _count()
    if out is not None:
        return out
    return res.view(*lead, D)


def _cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos, qk, sk, zk, qv, sv, zv, bits):
    B, G, n, D = key.shape
    ref_buf = k_buf if k_buf is not None else qk
    C = ref_buf.shape[2]
    for t in (k_buf, v_buf, token_pos, qk, sk, zk, qv, sv, zv):
        if t is not None and not t.is_contiguous():
            raise NativeError("cache_write: cache buffers must be contiguous")
    if k_buf is not None and k_buf.dtype != key.dtype:
        key, value = key.to(k_buf.dtype), value.to(k_buf.dtype)
    # rows of a (batch, group) D apart, the other strides free: a slice of positions of a longer tensor is read in place
    if not (key.stride(3) == 1 and key.stride(2) == D and key.stride() == value.stride()
            and key.stride(0) % 8 == 0 and key.stride(1) % 8 == 0):
        key, value = key.contiguous(), value.contiguous()
    if slots.dtype != torch.int32:
        slots = slots.to(torch.int32)
    if slots.stride(2) != 1:
        slots = slots.contiguous()
    st = status_word(key.device)
    _check(lib().kvb_cache_write_strided(_p(k_buf), _p(v_buf), _p(token_pos), _p(slots), _p(key), _p(value), _p(qk), _p(sk), _p(zk),
                                         _p(qv), _p(sv), _p(zv), B, G, n, D, C, _ll(slots.stride(0)), _ll(slots.stride(1)),
                                         _ll(key.stride(0)), _ll(key.stride(1)), int(input_pos), int(bits), _code(key.dtype), _p(st),
                                         _stream(key)), "cache_write")
    _count()


def cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos: int) -> None:
    _cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos, None, None, None, None, None, None, 0)


def cache_write_quant(k_buf, v_buf, token_pos, slots, key, value, input_pos, qk, sk, zk, qv, sv, zv, bits) -> None:
    _cache_write(k_buf, v_buf, token_pos, slots, key, value, input_pos, qk, sk, zk, qv, sv, zv, bits)


# ----------------------------------------------------------- gradient replay
def replay_supported(k_buf: torch.Tensor, key: torch.Tensor) -> bool:
    return (k_buf.is_cuda and k_buf.dtype == torch.bfloat16 and key.dtype == torch.bfloat16 and k_buf.shape[-1] == 128
            and k_buf.is_contiguous() and key.stride(-1) == 1 and all(st % 4 == 0 for st in key.stride()[:3]))


def replay_write(k_buf, v_buf, token_pos, slots, key, value, input_pos: int):
    """Saves what ``slots`` hold (returns ``old_k, old_v (B,G,n,D)``, ``old_tp (B,G,n)``), then writes
    ``key / value`` and the token positions ``input_pos + i`` there: one kernel."""
    B, G, n, D = key.shape
    C = k_buf.shape[2]
    if value.stride() != key.stride():
        value = value.contiguous()
        key = key.contiguous()
    slots = slots if slots.dtype == torch.int32 else slots.to(torch.int32)
    if slots.stride(2) != 1:
        slots = slots.contiguous()
    old_k = torch.empty((B, G, n, D), dtype=k_buf.dtype, device=k_buf.device)
    old_v = torch.empty_like(old_k)
    old_tp = torch.empty((B, G, n), dtype=torch.int32, device=k_buf.device)
    st = status_word(k_buf.device)
    _check(lib().kvb_replay_write(_p(k_buf), _p(v_buf), _p(token_pos), _p(slots), _p(key), _p(value), _p(old_k), _p(old_v), _p(old_tp),
                                  B, G, n, D, C, _ll(slots.stride(0)), _ll(slots.stride(1)), _ll(key.stride(0)), _ll(key.stride(1)),
                                  _ll(key.stride(2)), int(input_pos), _p(st), _stream(key)), "replay_write")
    _count()
    return old_k, old_v, old_tp


def replay_undo(k_buf, v_buf, token_pos, dk_buf, dv_buf, slots, old_k, old_v, old_tp):
    """Takes the accumulated gradients of the chunk's rows out of ``dk_buf / dv_buf`` (returned as
    bf16 ``(B,G,n,D)``, the slots are cleared) and restores the old content of the slots: one kernel."""
    B, G, n, D = old_k.shape
    C = k_buf.shape[2]
    slots = slots if slots.dtype == torch.int32 else slots.to(torch.int32)
    if slots.stride(2) != 1:
        slots = slots.contiguous()
    dk_new = torch.empty((B, G, n, D), dtype=k_buf.dtype, device=k_buf.device)
    dv_new = torch.empty_like(dk_new)
    st = status_word(k_buf.device)
    _check(lib().kvb_replay_undo(_p(k_buf), _p(v_buf), _p(token_pos), _p(dk_buf), _p(dv_buf), _p(slots), _p(old_k), _p(old_v),
                                 _p(old_tp), _p(dk_new), _p(dv_new), B, G, n, D, C, _ll(slots.stride(0)), _ll(slots.stride(1)),
                                 _p(st), _stream(old_k)), "replay_undo")
    _count()
    return dk_new, dv_new


# ---------------------------------------------------------------------- H2O
def h2o_update(scores, weights, k_select, n_evictable, normalize=False, token_pos=None, input_pos=0, prefill_length=0, out=None):
    """``weights`` may be ``None`` (selection only). ``out (B,G,k_select)`` int32 contiguous receives the
    result when given, so that a consumer captured in a CUDA graph reads a fixed address."""
    B, G, C = scores.shape
    if k_select > 4096 or (n_evictable * 4 + 8 * 2 ** math.ceil(math.log2(max(k_select, 2)))) > 200 * 1024:
        # cold path: full sort / very large selections stay with the library routine
        from keys_values_b200.ops import reference as ref

        res = ref.h2o_update(scores, weights, k_select, n_evictable, normalize, token_pos, input_pos, prefill_length)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if weights is not None:
        weights = weights.contiguous()
    if scores.stride(2) != 1:
        raise NativeError("h2o_update: scores must be contiguous along the slot axis")
    if out is None:
        out = torch.empty((B, G, k_select), dtype=torch.int32, device=scores.device)
    elif out.shape != (B, G, k_select) or out.dtype != torch.int32 or not out.is_contiguous():
        raise NativeError("h2o_update: out must be a contiguous int32 (B, G, k_select) tensor")
    tp = token_pos if normalize else None
    _check(lib().kvb_h2o_update(_p(scores), _p(weights), _p(tp), _p(out), B, G, C, n_evictable, k_select, int(normalize),
                                int(input_pos), int(prefill_length or 0), _ll(scores.stride(0)), _ll(scores.stride(1)),
                                _ll(tp.stride(0) if tp is not None else 0), _ll(tp.stride(1) if tp is not None else 0),
                                _stream(scores)), "h2o_update")
    _count()
    return out


# ------------------------------------------------- device-resident position (captured decode steps)
_POSITION: Optional["device_position"] = None


def position_context() -> Optional["device_position"]:
    """The active :class:`device_position` (``.word``: the int32 device word; ``.cache``: values derived
    from it once per step, e.g. the gathered RoPE rows), or ``None``."""
    return _POSITION


class device_position:
    """While active, cache writes and the H2O update read the position of the step's token from
    ``word`` (int32, one element, on the GPU) instead of their host argument, and the position
    encoding gathers its table row by it: a decode step captured in a CUDA graph then serves every
    later position (the graph increments the word itself)."""

    def __init__(self, word: torch.Tensor):
        if not (word.is_cuda and word.dtype == torch.int32 and word.numel() == 1):
            raise NativeError("device_position: need one int32 word on the GPU")
        self.word = word
        self.cache: dict = {}

    def __enter__(self):
        global _POSITION
        if _POSITION is not None:
            raise NativeError("device_position: already active")
        _POSITION = self
        lib().kvb_set_position_source.restype = None
        lib().kvb_set_position_source(_p(self.word))
        return self

    def __exit__(self, *exc):
        global _POSITION
        _POSITION = None
        lib().kvb_set_position_source(None)
        return False


# --------------------------------------------------------------------- GEMM
def gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0
            and x.stride(-1) == 1 and w.stride(-1) == 1)


def gemm(a: torch.Tensor, b: torch.Tensor, a2=None, b2=None, residual=None, out=None, max_ctas: int = 0) -> torch.Tensor:
    """``a (M,K) @ b (N,K)^T [+ a2 (M,K2) @ b2 (N,K2)^T] [+ residual (M,N)]`` in bf16 with fp32 accumulation."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    K2 = 0 if a2 is None else a2.shape[1]
    st = status_word(a.device)
    _check(lib().kvb_gemm_bf16(_p(a), _p(b), _p(a2), _p(b2), _p(out), _p(residual), M, N, K, K2, _ll(a.stride(0)), _ll(b.stride(0)),
                               _ll(a2.stride(0) if a2 is not None else 0), _ll(b2.stride(0) if b2 is not None else 0),
                               _ll(out.stride(0)), _p(st), int(max_ctas), _stream(a)), "gemm_bf16")
    _count()
    return out


def gemm_pair(a: torch.Tensor, b: torch.Tensor, a2=None, b2=None, residual=None, out=None, max_pairs: int = 0) -> torch.Tensor:
    """The same product as :func:`gemm` on CTA pairs (``tcgen05.mma.cta_group::2``, 256 x 256 tiles): each SM of a pair
    loads half of the B tile, which halves the shared-memory traffic per flop."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    K2 = 0 if a2 is None else a2.shape[1]
    st = status_word(a.device)
    _check(lib().kvb_gemm2_bf16(_p(a), _p(b), _p(a2), _p(b2), _p(out), _p(residual), M, N, K, K2, _ll(a.stride(0)), _ll(b.stride(0)),
                                _ll(a2.stride(0) if a2 is not None else 0), _ll(b2.stride(0) if b2 is not None else 0),
                                _ll(out.stride(0)), _p(st), int(max_pairs), _stream(a)), "gemm2_bf16")
    _count()
    return out


# ---------------------------------------------------------------- attention
def sdpa_supported(query: torch.Tensor, key: torch.Tensor, sliding_window, softcap) -> bool:
    H, G = query.shape[1], key.shape[1]
    gs = H // G
    return (query.dtype == torch.bfloat16 and query.shape[-1] in (64, 128, 256) and gs <= 128 and query.shape[2] > 0
            and (sliding_window is None or sliding_window > 0) and (softcap is None or softcap > 0))


def sdpa_bwd_supported(query: torch.Tensor, key: torch.Tensor, sliding_window, softcap) -> bool:
    """Same shapes as the forward, with at most 64 query heads per KV head (a 64-column unit of the dK/dV launch
    holds all heads of a group). Any group size: 5 (Qwen3-14B) packs 25 positions x 5 heads into the 128-row tile."""
    return (sdpa_supported(query, key, sliding_window, softcap) and query.shape[-1] in (64, 128)
            and query.shape[1] // key.shape[1] <= 64)


def sdpa_fwd(query, key, value, scale, input_pos, token_pos=None, return_weights=False, sliding_window=None, softcap=None):
    """SDPA forward: flash sweep (P in TMEM, online softmax) + column-owner weight sums. Returns
    ``(out (B,T,H·D) bf16, weights (B,G,L) fp32 | None, lse (B,H,T) fp32)``; head size 128, 64 or 256 (256: forward
    only, one query tile per CTA), any group size up to 128.
    ``sliding_window``: a query at position ``p`` sees tokens in ``(p - window, p]`` only; ``softcap``: scores
    become ``cap · tanh(score / cap)`` (both inside the kernels)."""
    B, H, T, D = query.shape
    G, L = key.shape[1], key.shape[2]
    query = _rows_in_place(query)
    if key.stride(3) != 1 or key.stride(2) != D or key.stride() != value.stride():
        key, value = key.contiguous(), value.contiguous()
    token_pos = _norm_token_pos(token_pos, B, G, L)
    dev = query.device
    out = torch.empty((B, T, H * D), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=dev)
    weights = torch.empty((B, G, L), dtype=torch.float32, device=dev) if return_weights else None
    lib().kvb_sdpa_fwd_scratch_bytes.restype = ctypes.c_longlong
    nbytes = lib().kvb_sdpa_fwd_scratch_bytes(B, H, G, T, L)
    if nbytes < 0:
        raise NativeError("sdpa_fwd: unsupported head / group configuration")
    scratch = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    st = status_word(dev)
    _check(lib().kvb_sdpa_fwd_ex(_p(query), _p(key), _p(value), _p(token_pos), _p(out), _p(lse), _p(weights), _p(scratch), B, H, G, T, L,
                                  int(D), _ll(query.stride(0)), _ll(query.stride(1)), _ll(key.stride(0)), _ll(key.stride(1)),
                                  _ll(token_pos.stride(0) if token_pos is not None else 0),
                                  _ll(token_pos.stride(1) if token_pos is not None else 0),
                                  ctypes.c_float(scale), int(input_pos), int(sliding_window or 0), ctypes.c_float(softcap or 0.0),
                                  _p(st), _stream(query)), "sdpa_fwd")
    _count(3 if return_weights else 2)
    return out, weights, lse


def _rows_in_place(query: torch.Tensor) -> torch.Tensor:
    """``query (B,H,T,D)`` as the attention kernels read it: rows of a head ``D`` apart, head and batch strides free
    (multiples of 8 elements), so that a slice of positions of a longer tensor is not copied; anything else is made
    contiguous."""
    D = query.shape[3]
    if (query.stride(3) == 1 and query.stride(2) == D and query.stride(1) % 8 == 0 and query.stride(0) % 8 == 0
            and query.stride(1) >= query.shape[2] * D and query.data_ptr() % 16 == 0):
        return query
    return query.contiguous()


def _norm_token_pos(token_pos, B, G, L):
    if token_pos is None:
        return None
    if token_pos.ndim == 1:
        token_pos = token_pos.view(1, 1, L).expand(B, G, L)
    if token_pos.dtype != torch.int32:
        token_pos = token_pos.to(torch.int32)
    if token_pos.stride(2) != 1:
        token_pos = token_pos.contiguous()
    return token_pos


def sdpa_bwd(grad_out, query, key, value, out, lse, scale, input_pos, token_pos=None, dk_accum=None, dv_accum=None,
             sliding_window=None, softcap=None):
    """Attention backward (tcgen05 kernels). Returns ``(dq, dk, dv)``: ``dq (B,H,T,D)`` in
    the dtype of ``query``; ``dk, dv`` fp32. If ``dk_accum/dv_accum`` (fp32, cache shaped,
    contiguous along the last two axes) are given, the gradients are *added* into their
    first ``kv_len`` slots and ``None`` is returned for them."""
    B, H, T, D = query.shape
    G, L = key.shape[1], key.shape[2]
    dev = query.device
    lib().kvb_sdpa_bwd_scratch_bytes.restype = ctypes.c_longlong
    query = _rows_in_place(query)
    grad_out = grad_out.contiguous()
    out = out.contiguous()
    if key.stride(3) != 1 or key.stride(2) != D or key.stride() != value.stride():
        key, value = key.contiguous(), value.contiguous()
    token_pos = _norm_token_pos(token_pos, B, G, L)
    own = dk_accum is None
    if own:
        dk_accum = torch.zeros((B, G, L, D), dtype=torch.float32, device=dev)
        dv_accum = torch.zeros((B, G, L, D), dtype=torch.float32, device=dev)
    elif dk_accum.stride(3) != 1 or dk_accum.stride(2) != D or dk_accum.stride() != dv_accum.stride() or dk_accum.dtype != torch.float32:
        raise NativeError("sdpa_bwd: accumulators must be fp32 with contiguous rows and equal strides")
    dq = torch.empty((B, H, T, D), dtype=torch.bfloat16, device=dev)
    nbytes = lib().kvb_sdpa_bwd_scratch_bytes(B, H, G, T, L)
    scratch = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    st = status_word(dev)
    _check(lib().kvb_sdpa_bwd_ex(_p(query), _p(key), _p(value), _p(token_pos), _p(out), _p(grad_out), _p(lse.contiguous()), _p(dq),
                                 _p(dk_accum), _p(dv_accum), _p(scratch), B, H, G, T, L, int(D), _ll(query.stride(0)), _ll(query.stride(1)),
                                 _ll(key.stride(0)), _ll(key.stride(1)),
                                 _ll(token_pos.stride(0) if token_pos is not None else 0),
                                 _ll(token_pos.stride(1) if token_pos is not None else 0),
                                 _ll(dk_accum.stride(0)), _ll(dk_accum.stride(1)), ctypes.c_float(scale), int(input_pos),
                                 int(sliding_window or 0), ctypes.c_float(softcap or 0.0), _p(st), _stream(query)), "sdpa_bwd")
    _count(4)
    if own:
        return dq, dk_accum, dv_accum
    return dq, None, None


# -------------------------------------------------------------------- decode
def decode_supported(query: torch.Tensor, n_query_groups: int) -> bool:
    H = query.shape[1]
    return (query.is_cuda and query.dtype == torch.bfloat16 and query.shape[-1] == 128 and query.shape[2] == 1
            and H % n_query_groups == 0 and H // n_query_groups <= 16)


def decode_attention(query, key, value, scale, kv_len, return_weights=False, quant=None, new_kv=None, softcap=None,
                     sliding_window=None, token_pos=None, query_pos: int = 0):
    """One-token attention. ``key/value``: bf16 ``(Bmax,G,C,D)`` buffers (``quant is None``) or
    uint8 code buffers with ``quant = (k_scale, k_zp, v_scale, v_zp, bits)``. ``new_kv =
    (k_new (B,G,D), v_new (B,G,D), slot (B,G) int32)`` substitutes one row in full precision.
    ``softcap``: scores become ``cap · tanh(score / cap)``. ``sliding_window`` with ``token_pos (Bmax,G,C)`` int32 and
    ``query_pos`` (the position of the query token; inside :class:`device_position` the kernel reads the device word
    instead): slots whose token is at or before ``query_pos - sliding_window`` are hidden.
    Returns ``(out (B,1,H·D), weights (B,G,kv_len) | None)``."""
    B, H, _, D = query.shape
    G, C = key.shape[1], key.shape[2]
    dev = query.device
    if not key.is_contiguous() or not value.is_contiguous():
        raise NativeError("decode_attention: cache buffers must be contiguous")
    lib().kvb_decode_scratch_bytes.restype = ctypes.c_longlong
    out = torch.empty((B, 1, H * D), dtype=torch.bfloat16, device=dev)
    weights = torch.empty((B, G, kv_len), dtype=torch.float32, device=dev) if return_weights else None
    scratch = torch.empty(lib().kvb_decode_scratch_bytes(B, H, kv_len) // 4, dtype=torch.float32, device=dev)
    if quant is None:
        ks = kz = vs = vz = None
        bits = 16
    else:
        ks, kz, vs, vz, bits = quant
    kn = vn = sl = None
    if new_kv is not None:
        kn, vn, sl = new_kv
        kn, vn = kn.contiguous(), vn.contiguous()
        sl = sl.to(torch.int32).contiguous()
    tp = None
    if sliding_window:
        if token_pos is None or token_pos.dtype != torch.int32 or token_pos.stride(2) != 1:
            raise NativeError("decode_attention: a sliding window needs int32 token positions (B, G, C) with unit stride")
        tp = token_pos
    _check(lib().kvb_decode_attn_ex(_p(query.contiguous()), _p(key), _p(value), _p(ks), _p(kz), _p(vs), _p(vz), _p(kn), _p(vn), _p(sl),
                                    _p(out), _p(weights), _p(scratch), B, H, G, int(kv_len), C, int(bits), ctypes.c_float(scale),
                                    ctypes.c_float(softcap or 0.0), int(sliding_window or 0), _p(tp),
                                    _ll(tp.stride(0) if tp is not None else 0), _ll(tp.stride(1) if tp is not None else 0),
                                    int(query_pos), _stream(query)), "decode_attn")
    _count(3 if return_weights else 2)
    return out, weights
