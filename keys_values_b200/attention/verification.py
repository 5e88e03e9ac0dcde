"""Equivalence of the sm_100a attention kernels with the fp32 restatement of the same operation.

The reference ships this as a user-facing check of its vendored FlashInfer kernels against the
eager implementation (``keys_values/attention/flashinfer_verification.py:32-377``); here the two
sides are ``ops.cuda.sdpa_fwd`` / ``ops.cuda.decode_attention`` (tcgen05 forward, MMA decode) and
``ops.reference.sdpa`` (plain PyTorch in fp32). Default tolerances are those of bf16 operands.
"""
from __future__ import annotations

import logging
from typing import Dict, List, Optional, Tuple

import torch

from keys_values_b200.ops import reference as ref

logger = logging.getLogger(__name__)


class BackendEquivalenceResult:
    """Outcome of one comparison; truthy when the outputs (and weights, if compared) agree."""

    def __init__(self, is_equivalent: bool, output_max_diff: float, output_mean_diff: float, weights_max_diff: Optional[float] = None,
                 weights_mean_diff: Optional[float] = None, rtol: float = 2e-2, atol: float = 2e-2, message: str = ""):
        self.is_equivalent = is_equivalent
        self.output_max_diff, self.output_mean_diff = output_max_diff, output_mean_diff
        self.weights_max_diff, self.weights_mean_diff = weights_max_diff, weights_mean_diff
        self.rtol, self.atol, self.message = rtol, atol, message

    def __bool__(self) -> bool:
        return self.is_equivalent

    def __repr__(self) -> str:
        fmt = lambda v: "None" if v is None else f"{v:.2e}"  # noqa: E731
        return (f"BackendEquivalenceResult(is_equivalent={self.is_equivalent}, output_max_diff={fmt(self.output_max_diff)}, "
                f"output_mean_diff={fmt(self.output_mean_diff)}, weights_max_diff={fmt(self.weights_max_diff)}, "
                f"weights_mean_diff={fmt(self.weights_mean_diff)})")


def check_numerical_equivalence(tensor_a: torch.Tensor, tensor_b: torch.Tensor, rtol: float = 2e-2, atol: float = 2e-2) -> Tuple[bool, float, float]:
    """``(allclose, max |a − b|, mean |a − b|)`` in fp32."""
    if tensor_a.shape != tensor_b.shape:
        raise ValueError(f"Shape mismatch: {tuple(tensor_a.shape)} vs {tuple(tensor_b.shape)}")
    a, b = tensor_a.float(), tensor_b.float()
    diff = (a - b).abs()
    return bool(torch.allclose(a, b, rtol=rtol, atol=atol)), float(diff.max()), float(diff.mean())


def verify_backend_equivalence(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale_factor: float,
                               return_attn_weights: bool = False, token_positions: Optional[torch.Tensor] = None, input_pos: int = 0,
                               rtol: float = 2e-2, atol: float = 2e-2, log_results: bool = True,
                               sliding_window_size: Optional[int] = None, softcap: Optional[float] = None) -> BackendEquivalenceResult:
    """``query (B,H,q,D)``, ``key / value (B,G,kv,D)`` on a GPU. A query of length 1 goes to the decode
    kernel, longer ones (and layers with a sliding window or capped scores) to the tcgen05 forward (head size 128,
    64 or 256); the weights compared are the per-slot sums the
    cache policies consume (``(B,G,kv)``, summed over queries, averaged over the heads of a group)."""
    from keys_values_b200.ops import cuda as cu

    if not query.is_cuda:
        raise RuntimeError("the kernels run on a GPU; the tensors are on " + str(query.device))
    B, H, T, D = query.shape
    L = key.shape[2]
    if T == 1 and token_positions is None and sliding_window_size is None and softcap is None and cu.decode_supported(query, key.shape[1]):
        out, w = cu.decode_attention(query, key.contiguous(), value.contiguous(), scale_factor, L, return_attn_weights)
    elif cu.sdpa_supported(query, key, sliding_window_size, softcap):
        out, w, _ = cu.sdpa_fwd(query, key, value, scale_factor, input_pos, token_positions, return_attn_weights,
                                sliding_window_size, softcap)
    else:
        raise RuntimeError(f"no kernel for query {tuple(query.shape)} {query.dtype}, key {tuple(key.shape)}")
    cu.check_status(query.device)
    res = ref.sdpa(query, key, value, scale_factor, input_pos, token_positions, return_attn_weights, sliding_window_size, softcap)
    out_r, w_r = res[0], res[1]
    ok, omax, omean = check_numerical_equivalence(out, out_r.to(out.dtype), rtol, atol)
    wmax = wmean = None
    if return_attn_weights:
        okw, wmax, wmean = check_numerical_equivalence(w, w_r, rtol, max(atol * 1e-1, 1e-3))
        ok = ok and okw
    msg = ("equivalent" if ok else "NOT equivalent") + f": B={B} H={H} q={T} kv={L} D={D}"
    if log_results:
        (logger.info if ok else logger.warning)("%s (output max diff %.2e)", msg, omax)
    return BackendEquivalenceResult(ok, omax, omean, wmax, wmean, rtol, atol, msg)


def verify_backend_equivalence_batch(test_cases: List[Dict], rtol: float = 2e-2, atol: float = 2e-2, log_results: bool = True,
                                     stop_on_failure: bool = False) -> Tuple[int, int, List[BackendEquivalenceResult]]:
    """Each case: ``query, key, value, scale_factor`` and optionally ``return_attn_weights,
    token_positions, input_pos``. Returns ``(passed, failed, results)``."""
    results: List[BackendEquivalenceResult] = []
    for case in test_cases:
        results.append(verify_backend_equivalence(rtol=rtol, atol=atol, log_results=log_results, **case))
        if stop_on_failure and not results[-1]:
            break
    passed = sum(bool(r) for r in results)
    return passed, len(results) - passed, results
