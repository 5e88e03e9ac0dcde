"""The allocation-free decode entry point, called through its exported C symbol.

Callers that cannot create device memory at call time (a frozen allocator, a serving loop with
a fixed memory plan, a foreign-language host that only links the C API) use
``kvb_decode_attn_noalloc``; its workspace is a fixed array inside the library. The test checks
it against the regular entry point, which takes a caller-provided workspace, on two calls in
a row (the second call reuses the workspace left behind by the first), and checks that a
problem beyond the fixed size is refused.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def test_noalloc_decode_matches_regular_entry_point_twice():
    from keys_values_b200.ops import cuda as cu
    from keys_values_b200.ops import reference as ref

    lib = cu.lib()
    lib.kvb_decode_attn_noalloc_max_bytes.restype = ctypes.c_longlong
    lib.kvb_decode_scratch_bytes.restype = ctypes.c_longlong
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, H, G, L, C, D = 2, 32, 8, 3000, 4096, 128
    assert lib.kvb_decode_scratch_bytes(B, H, L) <= lib.kvb_decode_attn_noalloc_max_bytes()
    scale = 1.0 / math.sqrt(D)
    gen = torch.Generator(device=dev).manual_seed(5)
    for call in range(2):
        L_call = L - 700 * call  # the second call has another size: it must not depend on leftovers
        q = torch.randn(B, H, 1, D, device=dev, dtype=torch.bfloat16, generator=gen)
        k = torch.randn(B, G, C, D, device=dev, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(B, G, C, D, device=dev, dtype=torch.bfloat16, generator=gen)
        qk, sk, zk = ref.quantize_rows(k, 8)
        qv, sv, zv = ref.quantize_rows(v, 8)
        out_ref, w_ref = cu.decode_attention(q, qk, qv, scale, L_call, True, quant=(sk, zk, sv, zv, 8))
        out = torch.empty_like(out_ref)
        w = torch.empty_like(w_ref)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        rc = lib.kvb_decode_attn_noalloc(_p(q), _p(qk), _p(qv), _p(sk), _p(zk), _p(sv), _p(zv), _p(None), _p(None), _p(None), _p(out), _p(w),
                                         B, H, G, L_call, C, 8, ctypes.c_float(scale), stream)
        assert rc == 0
        torch.cuda.synchronize(dev)
        torch.testing.assert_close(out.float(), out_ref.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(w, w_ref, atol=1e-3, rtol=2e-2)


def test_noalloc_decode_refuses_oversized_problem():
    from keys_values_b200.ops import cuda as cu

    lib = cu.lib()
    lib.kvb_decode_attn_noalloc_max_bytes.restype = ctypes.c_longlong
    lib.kvb_decode_scratch_bytes.restype = ctypes.c_longlong
    B, H, L = 8, 32, 32768
    assert lib.kvb_decode_scratch_bytes(B, H, L) > lib.kvb_decode_attn_noalloc_max_bytes()
    null = ctypes.c_void_p(0)
    rc = lib.kvb_decode_attn_noalloc(null, null, null, null, null, null, null, null, null, null, null, null, B, H, 8, L, L, 8,
                                     ctypes.c_float(1.0), null)
    assert rc == -7  # KVB_ERR_TOO_LARGE: nothing was launched
