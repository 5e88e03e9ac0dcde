"""Numerics of every CUDA kernel against the plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

from keys_values_b200 import ops
from keys_values_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cuda():
    from keys_values_b200.ops import cuda

    return cuda


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,dim,unit", [(37, 2560, False), (8, 64, True), (300, 1000, False)])
def test_rmsnorm(dtype, rows, dim, unit):
    x = torch.randn(rows, dim, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(dim, device=DEV, dtype=dtype) * 0.1 + 1.0).requires_grad_(True)
    y = ops.rmsnorm(x, w, 1e-6, unit)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = ref.rmsnorm(xr, wr, 1e-6, unit)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(y.float(), yr, atol=tol, rtol=tol)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=tol * 2, rtol=tol * 2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=tol * 8, rtol=tol * 4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,H,G,D,rope,norm", [(2, 33, 8, 2, 128, 128, True), (1, 16, 4, 4, 64, 32, False), (1, 7, 4, 2, 16, 16, True)])
def test_qknorm_rope(dtype, B, T, H, G, D, rope, norm):
    qkv = torch.randn(B, T, (H + 2 * G) * D, device=DEV, dtype=dtype, requires_grad=True)
    pos = torch.arange(T, device=DEV).float()[:, None] * torch.rand(rope // 2, device=DEV)[None]
    ang = torch.cat((pos, pos), -1)
    cos, sin = ang.cos(), ang.sin()
    qw = (torch.rand(D, device=DEV, dtype=dtype) + 0.5).requires_grad_(True) if norm else None
    kw = (torch.rand(D, device=DEV, dtype=dtype) + 0.5).requires_grad_(True) if norm else None
    q, k, v = ops.qknorm_rope(qkv, H, G, D, cos, sin, qw, kw, 1e-6, rope)
    qkv_r = qkv.detach().float().requires_grad_(True)
    qw_r = qw.detach().float().requires_grad_(True) if norm else None
    kw_r = kw.detach().float().requires_grad_(True) if norm else None
    qr, kr, vr = ref.qknorm_rope(qkv_r, H, G, D, cos, sin, qw_r, kw_r, 1e-6, rope)
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-5
    for a, b in ((q, qr), (k, kr), (v, vr)):
        torch.testing.assert_close(a.float(), b, atol=tol, rtol=tol)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    torch.testing.assert_close(qkv.grad.float(), qkv_r.grad, atol=tol * 2, rtol=tol * 2)
    if norm:
        torch.testing.assert_close(qw.grad.float(), qw_r.grad, atol=tol * 16, rtol=tol * 4)
        torch.testing.assert_close(kw.grad.float(), kw_r.grad, atol=tol * 16, rtol=tol * 4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    a = torch.randn(5, 1003, device=DEV, dtype=dtype, requires_grad=True)
    b = torch.randn(5, 1003, device=DEV, dtype=dtype, requires_grad=True)
    y = ops.swiglu(a, b)
    ar, br = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = ref.swiglu(ar, br)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(y.float(), yr, atol=tol, rtol=tol)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(a.grad.float(), ar.grad, atol=tol * 2, rtol=tol * 2)
    torch.testing.assert_close(b.grad.float(), br.grad, atol=tol * 2, rtol=tol * 2)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quantize_roundtrip(bits, dtype):
    x = torch.randn(2, 3, 50, 128, device=DEV, dtype=dtype)
    q, s, z = ops.quantize_rows(x, bits)
    qr, sr, zr = ref.quantize_rows(x, bits)
    torch.testing.assert_close(s, sr)
    assert (z - zr).abs().max().item() <= 1 and ((z - zr) != 0).float().mean().item() < 2e-2
    # codes agree wherever the zero points agree, up to rounding ties of x/scale (the library
    # division may differ in the last ulp); a zero point that differs by one shifts its whole row
    same_row = (z == zr).unsqueeze(-1)
    if bits == 8:
        diff = (q.int() - qr.int()).abs()
    else:
        diff = torch.maximum(((q >> 4).int() - (qr >> 4).int()).abs(), ((q & 15).int() - (qr & 15).int()).abs())
    assert diff.max().item() <= 1 and ((diff > 0) & same_row).float().mean().item() < 2e-3
    d = ops.dequantize_rows(q, s, z, bits, dtype)
    dr = ref.dequantize_rows(q, s, z, bits, dtype)
    # round trip error is bounded by the quantization step
    assert ((d.float() - x.float()).abs() <= 1.01 * s.unsqueeze(-1) + 1e-6).all()
    torch.testing.assert_close(d.float(), dr.float(), atol=1e-6, rtol=1e-6)
    # strided destination (a slot range of a larger buffer)
    buf = torch.zeros(2, 3, 80, 128, device=DEV, dtype=dtype)
    ops.dequantize_rows(q, s, z, bits, dtype, out=buf[:, :, :50])
    torch.testing.assert_close(buf[:, :, :50].float(), dr.float(), atol=1e-6, rtol=1e-6)
    assert buf[:, :, 50:].abs().max().item() == 0


@pytest.mark.parametrize("sliced", [False, True])
@pytest.mark.parametrize("bits", [0, 8, 4])
def test_cache_write(bits, sliced):
    B, G, C, D, n = 2, 3, 40, 128, 7
    dt = torch.bfloat16
    kb = torch.randn(B, G, C, D, device=DEV, dtype=dt)
    vb = torch.randn(B, G, C, D, device=DEV, dtype=dt)
    tp = torch.zeros(B, G, C, device=DEV, dtype=torch.int32)
    slots = torch.stack([torch.stack([torch.randperm(C, device=DEV)[:n] for _ in range(G)]) for _ in range(B)]).to(torch.int32)
    key, val = torch.randn(B, G, n, D, device=DEV, dtype=dt), torch.randn(B, G, n, D, device=DEV, dtype=dt)
    if sliced:  # the rows of a chunk inside the cell's longer tensor: read through the batch and group strides, no copy
        key = torch.randn(B, G, 3 * n, D, device=DEV, dtype=dt)[:, :, n:2 * n]
        val = torch.randn(B, G, 3 * n, D, device=DEV, dtype=dt)[:, :, n:2 * n]
        assert not key.is_contiguous()
    kb_r, vb_r, tp_r = kb.clone(), vb.clone(), tp.clone()
    ref.cache_write(kb_r, vb_r, tp_r, slots, key, val, 100)
    if bits == 0:
        ops.cache_write(kb, vb, tp, slots, key, val, 100)
    else:
        Dq = D if bits == 8 else D // 2
        qk = torch.zeros(B, G, C, Dq, device=DEV, dtype=torch.uint8); qv = torch.zeros_like(qk)
        sk = torch.ones(B, G, C, device=DEV); sv = torch.ones_like(sk)
        zk = torch.zeros(B, G, C, device=DEV, dtype=torch.int32); zv = torch.zeros_like(zk)
        ops.cache_write_quant(kb, vb, tp, slots, key, val, 100, qk, sk, zk, qv, sv, zv, bits)
        q_r, s_r, z_r = ref.quantize_rows(key, bits)
        idx = slots.long()
        torch.testing.assert_close(sk.gather(2, idx), s_r)
        assert (zk.gather(2, idx) - z_r).abs().max().item() <= 1
        got = qk.gather(2, idx.unsqueeze(-1).expand(-1, -1, -1, Dq))
        if bits == 8:
            dq = (got.int() - q_r.int()).abs()
        else:
            dq = torch.maximum(((got >> 4).int() - (q_r >> 4).int()).abs(), ((got & 15).int() - (q_r & 15).int()).abs())
        assert dq.max().item() <= 1 and (dq > 0).float().mean().item() < 2e-3
    torch.testing.assert_close(kb, kb_r)
    torch.testing.assert_close(vb, vb_r)
    torch.testing.assert_close(tp, tp_r)
    _cuda().check_status(DEV)


@pytest.mark.parametrize("C,k,normalize", [(512, 64, False), (16384, 1024, False), (1000, 100, True), (16384, 8, False), (777, 1, True),
                                           (4096, 32, True)])
def test_h2o_update(C, k, normalize):
    B, G = 2, 4
    scores = torch.rand(B, G, C, device=DEV)
    w = torch.rand(B, G, C, device=DEV)
    tp = torch.stack([torch.stack([torch.randperm(C, device=DEV) for _ in range(G)]) for _ in range(B)]).to(torch.int32)
    n_ev = C - 16
    s_r = scores.clone()
    idx_r = ref.h2o_update(s_r, w, k, n_ev, normalize, tp, C + 5, 17)
    idx = ops.h2o_update(scores, w, k, n_ev, normalize, tp, C + 5, 17)
    torch.testing.assert_close(scores, s_r)
    assert torch.equal(idx.sort(-1)[0], idx_r.sort(-1)[0])
    sel = s_r[:, :, :n_ev]
    if normalize:
        sel = sel / (C + 5 - tp[:, :, :n_ev].clamp(min=16)).float()
    vals = sel.gather(2, idx.long())
    assert (vals[:, :, 1:] >= vals[:, :, :-1]).all()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 6144, 2560), (200, 264, 136), (4096, 2560, 9728)])
def test_gemm(M, N, K):
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    c = _cuda().gemm(a, b)
    _cuda().check_status(DEV)
    cr = a.float() @ b.float().t()
    torch.testing.assert_close(c.float(), cr, atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 512), (1024, 6144, 2560), (200, 264, 136), (130, 520, 72), (4096, 2560, 9728)])
def test_gemm_on_cta_pairs(M, N, K):
    """The cta_group::2 kernel (256 x 256 tiles over two SMs), ragged edges included."""
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    c = _cuda().gemm_pair(a, b)
    _cuda().check_status(DEV)
    cr = a.float() @ b.float().t()
    torch.testing.assert_close(c.float(), cr, atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


def test_gemm_on_cta_pairs_wide_tiles():
    """Long K and many tiles: the launcher takes 256 x 512 tiles per pair (both accumulators of an SM in one tile)."""
    M, N, K = 8192, 8192, 4096  # 32 x 16 wide tiles: seven nearly full waves of 74 pairs
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    c = _cuda().gemm_pair(a, b)
    _cuda().check_status(DEV)
    cr = a.float() @ b.float().t()
    torch.testing.assert_close(c.float(), cr, atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


def test_gemm_on_cta_pairs_lora_residual():
    M, N, K, R = 512, 1024, 512, 64
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    a2 = torch.randn(M, R, device=DEV, dtype=torch.bfloat16)
    b2 = torch.randn(N, R, device=DEV, dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    c = _cuda().gemm_pair(a, b, a2, b2, residual=res)
    _cuda().check_status(DEV)
    cr = a.float() @ b.float().t() + a2.float() @ b2.float().t() + res.float()
    torch.testing.assert_close(c.float(), cr, atol=1e-1, rtol=2e-2)


def test_gemm_lora_residual():
    M, N, K, R = 512, 1024, 512, 64
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    a2 = torch.randn(M, R, device=DEV, dtype=torch.bfloat16)
    b2 = torch.randn(N, R, device=DEV, dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    c = _cuda().gemm(a, b, a2, b2, residual=res)
    _cuda().check_status(DEV)
    cr = a.float() @ b.float().t() + a2.float() @ b2.float().t() + res.float()
    torch.testing.assert_close(c.float(), cr, atol=1e-1, rtol=2e-2)


def _sdpa_case(B, H, G, T, L, input_pos, mode, want_w=True, window=None, softcap=None, D=128):
    q = torch.randn(B, H, T, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    if mode == "arange":
        tp = None
    else:
        # an evicted cache: distinct token positions; the last T tokens of the sequence are present
        tp = torch.empty(B, G, L, device=DEV, dtype=torch.int32)
        for b in range(B):
            for g in range(G):
                old = torch.randperm(input_pos, device=DEV)[: L - T]
                new = torch.arange(input_pos, input_pos + T, device=DEV)
                allp = torch.cat((old, new))
                tp[b, g] = allp[torch.randperm(L, device=DEV)].to(torch.int32)
    scale = 1.0 / math.sqrt(D)
    out, w, lse = _cuda().sdpa_fwd(q, k, v, scale, input_pos, tp, want_w, window, softcap)
    _cuda().check_status(DEV)
    out_r, w_r, lse_r = ref.sdpa(q, k, v, scale, input_pos, tp, want_w, window, softcap, return_lse=True)
    torch.testing.assert_close(lse, lse_r, atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(out.float(), out_r.float(), atol=2e-2, rtol=2e-2)
    if want_w:
        torch.testing.assert_close(w, w_r, atol=2e-2, rtol=2e-2)


def test_sdpa_single_tile():
    _sdpa_case(1, 4, 1, 32, 128, 96, "arange")


def test_sdpa_prefill_causal():
    _sdpa_case(1, 8, 2, 512, 512, 0, "arange", want_w=False)


@pytest.mark.parametrize("B,H,G,T,L", [(1, 32, 8, 256, 4096), (2, 8, 2, 100, 1000), (1, 4, 4, 64, 300), (1, 16, 2, 50, 777)])
def test_sdpa_evicted_cache(B, H, G, T, L):
    _sdpa_case(B, H, G, T, L, 5 * L, "perm")


def test_sdpa_group_size_not_a_power_of_two():
    # 40 query heads over 8 KV heads (Qwen3-14B): 25 positions x 5 heads fill 125 of the 128 tile rows
    _sdpa_case(1, 40, 8, 200, 1024, 5000, "perm")
    _sdpa_case(1, 10, 2, 77, 300, 0, "arange", want_w=False)


def test_sdpa_long_chunk_over_full_cache():
    # the training shape: 1024 new tokens scattered over a cache of 16384 slots
    _sdpa_case(1, 32, 8, 1024, 16384, 5 * 16384, "perm")


@pytest.mark.parametrize("B,H,G,T,L,mode", [(1, 8, 2, 100, 3000, "perm"), (1, 4, 1, 64, 8192, "perm"), (1, 5, 1, 60, 4100, "perm"),
                                             (1, 8, 2, 128, 2048, "arange")])
def test_sdpa_few_queries_split_over_the_cache(B, H, G, T, L, mode):
    """Few query tiles and a long cache: the flash sweep is split over the KV axis (several CTAs per query-tile
    pair, fp32 partials, a merge in a fixed order); one tensor-parallel rank with a single KV group is the typical case."""
    _sdpa_case(B, H, G, T, L, 4 * L if mode == "perm" else L - T, mode)


def test_sdpa_plain_causal_with_weights():
    # square causal prefill with weights: diagonal tiles take the element-wise mask path
    _sdpa_case(2, 8, 2, 700, 700, 0, "arange")


WINDOW_SOFTCAP_CASES = [
    (1, 8, 2, 300, 1500, "arange", 256, None),    # window edge inside the chunk's diagonal and before it
    (1, 8, 2, 300, 1500, "arange", None, 2.0),    # a cap that bends most scores
    (2, 8, 2, 100, 1000, "perm", 2500, 50.0),     # evicted cache: part of the old tokens outside the window
    (1, 10, 2, 77, 900, "arange", 100, 3.0),      # group size 5
    (1, 32, 8, 1, 2048, "arange", 512, 50.0),     # one query: a decode step of such a layer
    (1, 4, 1, 64, 8192, "arange", 1000, None),    # few queries: split over the KV axis, most tiles outside the window
    (1, 8, 2, 700, 700, "arange", 128, None),     # square prefill: a band of diagonal tiles
]


@pytest.mark.parametrize("B,H,G,T,L,mode,window,softcap", WINDOW_SOFTCAP_CASES)
def test_sdpa_sliding_window_and_softcap(B, H, G, T, L, mode, window, softcap):
    """Sliding window and logit soft-capping inside the tcgen05 kernels (outputs, normalisers, summed weights)."""
    _sdpa_case(B, H, G, T, L, 3 * L if mode == "perm" else L - T, mode, window=window, softcap=softcap)


@pytest.mark.parametrize("B,H,G,T,L,mode,window,softcap", [
    (1, 8, 2, 256, 2048, "perm", None, None), (2, 8, 2, 100, 1000, "perm", None, None), (1, 14, 2, 77, 900, "arange", None, None),
    (1, 32, 8, 700, 700, "arange", None, None), (1, 4, 1, 64, 8192, "perm", None, None), (1, 8, 2, 300, 1500, "arange", 256, 3.0),
    (1, 32, 8, 1, 2048, "arange", None, None)])
def test_sdpa_head_size_64(B, H, G, T, L, mode, window, softcap):
    """Head size 64 (Llama-3.2-1B, Qwen2.5-0.5B): tiles of one 64-feature chunk, O of 64 TMEM columns."""
    _sdpa_case(B, H, G, T, L, 3 * L if mode == "perm" else L - T, mode, window=window, softcap=softcap, D=64)


@pytest.mark.parametrize("D", [128, 64])
def test_sdpa_reads_a_slice_of_positions_in_place(D):
    """The queries of a chunk are a slice of the cell's (B,H,T',D) tensor: forward and backward read it through the
    head and batch strides (no copy) and give what the contiguous copy gives, bit for bit."""
    B, H, G, T, L, T_cell = 2, 8, 2, 200, 1000, 700
    q_cell = torch.randn(B, H, T_cell, D, device=DEV, dtype=torch.bfloat16)
    q = q_cell[:, :, 300:300 + T]
    assert not q.is_contiguous()
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    go = torch.randn(B, T, H * D, device=DEV, dtype=torch.bfloat16)
    scale, ip = 1.0 / math.sqrt(D), L - T
    res = []
    for qq in (q, q.contiguous()):
        out, w, lse = _cuda().sdpa_fwd(qq, k, v, scale, ip, None, True)
        dq, dk, dv = _cuda().sdpa_bwd(go, qq, k, v, out, lse, scale, ip, None)
        res.append((out, w, lse, dq, dk, dv))
    _cuda().check_status(DEV)
    for a, b in zip(*res):
        assert torch.equal(a, b)
    out_r, w_r, _ = ref.sdpa(q, k, v, scale, ip, None, True, return_lse=True)
    torch.testing.assert_close(res[0][0].float(), out_r.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("B,H,G,T,L,mode,window,softcap", [
    (1, 8, 4, 256, 2048, "perm", None, None), (2, 8, 4, 100, 1000, "perm", None, None), (1, 16, 8, 700, 700, "arange", None, None),
    (1, 8, 4, 300, 1500, "arange", 256, 50.0), (1, 4, 1, 64, 8192, "perm", None, None), (1, 8, 4, 1, 2048, "arange", 512, 50.0),
    (1, 6, 2, 77, 900, "arange", None, None)])
def test_sdpa_head_size_256(B, H, G, T, L, mode, window, softcap):
    """Head size 256 (Gemma-2 2b / 9b, Gemma-3 shapes), forward: one query tile per CTA, S double buffered over the KV
    tiles, O of 256 TMEM columns; outputs, normalisers and summed weights."""
    _sdpa_case(B, H, G, T, L, 3 * L if mode == "perm" else L - T, mode, window=window, softcap=softcap, D=256)


def test_sdpa_is_deterministic():
    """Outputs, normalisers and the summed weights (which drive the eviction decisions) are bit-identical run to run."""
    D, B, H, G, T, L = 128, 1, 32, 8, 512, 4096  # 64 CTAs: split over the KV axis, partials merged in a fixed order
    q = torch.randn(B, H, T, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    tp = torch.stack([torch.stack([torch.randperm(L, device=DEV) for _ in range(G)]) for _ in range(B)]).to(torch.int32) + 3 * L
    tp[:, :, ::8][:, :, :T] = (torch.arange(T, device=DEV) + 5 * L).to(torch.int32)  # the chunk's tokens, scattered
    runs = [_cuda().sdpa_fwd(q, k, v, 1 / math.sqrt(D), 5 * L, tp, True) for _ in range(3)]
    _cuda().check_status(DEV)
    for r in runs[1:]:
        assert torch.equal(r[0], runs[0][0]) and torch.equal(r[1], runs[0][1]) and torch.equal(r[2], runs[0][2])
    # the k smallest scores (the slots H2O would evict) agree as index sets as well
    idx = [torch.topk(r[1], 64, largest=False).indices.sort(dim=-1).values for r in runs]
    assert all(torch.equal(i, idx[0]) for i in idx[1:])


def test_sdpa_status_reports_timeout_free_run():
    # a healthy run leaves the status word at zero
    _sdpa_case(1, 4, 1, 32, 256, 224, "arange")
    assert int(_cuda().status_word(DEV).item()) == 0


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("B,H,G,T,L,mode", [(1, 4, 1, 32, 128, "arange"), (1, 8, 2, 256, 256, "prefill"), (2, 8, 2, 100, 1000, "perm"),
                                             (1, 32, 8, 256, 2048, "perm"), (1, 4, 4, 64, 300, "perm"),
                                             (1, 10, 2, 100, 700, "perm"), (2, 7, 1, 64, 300, "arange"), (1, 40, 8, 130, 1024, "perm"),
                                             (1, 3, 1, 50, 200, "perm"), (1, 12, 2, 77, 500, "perm")])  # group sizes 5, 7, 3, 6: rows and columns of a tile not all used
def test_sdpa_bwd(B, H, G, T, L, mode):
    if mode == "prefill":
        mode = "arange"
    D = 128
    q = torch.randn(B, H, T, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    go = torch.randn(B, T, H * D, device=DEV, dtype=torch.bfloat16)
    if mode == "perm":
        input_pos = 3 * L
        tp = torch.empty(B, G, L, device=DEV, dtype=torch.int32)
        for b in range(B):
            for g in range(G):
                allp = torch.cat((torch.randperm(input_pos, device=DEV)[: L - T], torch.arange(input_pos, input_pos + T, device=DEV)))
                tp[b, g] = allp[torch.randperm(L, device=DEV)].to(torch.int32)
    else:
        tp = None
        input_pos = L - T
    scale = 1.0 / math.sqrt(D)
    out, _, lse = _cuda().sdpa_fwd(q, k, v, scale, input_pos, tp, False)
    # accumulate into a larger cache-shaped buffer that already holds something
    C = L + 40
    dk_acc = torch.randn(B, G, C, D, device=DEV)
    dv_acc = torch.randn(B, G, C, D, device=DEV)
    dk0, dv0 = dk_acc.clone(), dv_acc.clone()
    dq, _, _ = _cuda().sdpa_bwd(go, q, k, v, out, lse, scale, input_pos, tp, dk_acc, dv_acc)
    _cuda().check_status(DEV)
    dq_r, dk_r, dv_r = ref.sdpa_backward(go, q, k, v, scale, input_pos, tp)
    assert _rel_err(dq, dq_r) < 3e-2
    assert _rel_err(dk_acc[:, :, :L] - dk0[:, :, :L], dk_r) < 3e-2
    assert _rel_err(dv_acc[:, :, :L] - dv0[:, :, :L], dv_r) < 3e-2
    assert torch.equal(dk_acc[:, :, L:], dk0[:, :, L:]) and torch.equal(dv_acc[:, :, L:], dv0[:, :, L:])


@pytest.mark.parametrize("B,H,G,T,L,mode,window,softcap", [
    (1, 8, 2, 256, 2048, "perm", None, None), (2, 8, 2, 100, 1000, "perm", None, None), (1, 14, 2, 77, 900, "arange", None, None),
    (1, 32, 8, 700, 700, "arange", None, None), (1, 3, 1, 50, 200, "perm", None, None), (1, 8, 2, 300, 1500, "arange", 256, 3.0)])
def test_sdpa_bwd_head_size_64(B, H, G, T, L, mode, window, softcap):
    test_sdpa_bwd_sliding_window_and_softcap(B, H, G, T, L, mode, window, softcap, D=64)


@pytest.mark.parametrize("B,H,G,T,L,mode,window,softcap", WINDOW_SOFTCAP_CASES)
def test_sdpa_bwd_sliding_window_and_softcap(B, H, G, T, L, mode, window, softcap, D=128):
    q = torch.randn(B, H, T, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    go = torch.randn(B, T, H * D, device=DEV, dtype=torch.bfloat16)
    if mode == "perm":
        input_pos = 3 * L
        tp = torch.empty(B, G, L, device=DEV, dtype=torch.int32)
        for b in range(B):
            for g in range(G):
                allp = torch.cat((torch.randperm(input_pos, device=DEV)[: L - T], torch.arange(input_pos, input_pos + T, device=DEV)))
                tp[b, g] = allp[torch.randperm(L, device=DEV)].to(torch.int32)
    else:
        tp, input_pos = None, L - T
    scale = 1.0 / math.sqrt(D)
    out, _, lse = _cuda().sdpa_fwd(q, k, v, scale, input_pos, tp, False, window, softcap)
    dq, dk, dv = _cuda().sdpa_bwd(go, q, k, v, out, lse, scale, input_pos, tp, sliding_window=window, softcap=softcap)
    _cuda().check_status(DEV)
    dq_r, dk_r, dv_r = ref.sdpa_backward(go, q, k, v, scale, input_pos, tp, window, softcap)
    assert _rel_err(dq, dq_r) < 3e-2
    assert _rel_err(dk, dk_r) < 3e-2
    assert _rel_err(dv, dv_r) < 3e-2


@pytest.mark.parametrize("bits", [16, 8, 4])
@pytest.mark.parametrize("B,H,G,L,C", [(1, 32, 8, 4096, 4096), (2, 8, 2, 1500, 2048), (1, 4, 4, 100, 128), (2, 14, 2, 777, 1024),
                                       (1, 32, 2, 300, 512)])
def test_decode_attention(bits, B, H, G, L, C):
    D = 128
    scale = 1.0 / math.sqrt(D)
    q = torch.randn(B, H, 1, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16)
    if bits == 16:
        out, w = _cuda().decode_attention(q, k, v, scale, L, True)
        k_eff, v_eff = k[:, :, :L], v[:, :, :L]
    else:
        qk, sk, zk = ref.quantize_rows(k, bits)
        qv, sv, zv = ref.quantize_rows(v, bits)
        slot = torch.randint(0, L, (B, G), device=DEV, dtype=torch.int32)
        k_new = torch.randn(B, G, D, device=DEV, dtype=torch.bfloat16)
        v_new = torch.randn(B, G, D, device=DEV, dtype=torch.bfloat16)
        out, w = _cuda().decode_attention(q, qk, qv, scale, L, True, quant=(sk, zk, sv, zv, bits), new_kv=(k_new, v_new, slot))
        k_eff = ref.dequantize_rows(qk, sk, zk, bits, torch.bfloat16)[:, :, :L].clone()
        v_eff = ref.dequantize_rows(qv, sv, zv, bits, torch.bfloat16)[:, :, :L].clone()
        idx = slot.long().view(B, G, 1, 1).expand(B, G, 1, D)
        k_eff.scatter_(2, idx, k_new.unsqueeze(2))
        v_eff.scatter_(2, idx, v_new.unsqueeze(2))
    out_r, w_r = ref.sdpa(q, k_eff, v_eff, scale, L - 1, None, True)
    torch.testing.assert_close(out.float(), out_r.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(w, w_r, atol=1e-3, rtol=2e-2)


@pytest.mark.parametrize("bits", [16, 8, 4])
@pytest.mark.parametrize("B,H,G,L,C,window,softcap", [(1, 32, 8, 4096, 4096, 1000, None), (2, 8, 2, 1500, 2048, None, 2.0),
                                                      (2, 14, 2, 777, 1024, 300, 3.0)])
def test_decode_attention_sliding_window_and_softcap(bits, B, H, G, L, C, window, softcap):
    """The decode kernel with capped scores and with slots hidden by a sliding window (an evicted cache: the tokens
    of the slots are a random subset of the positions before the query)."""
    D = 128
    scale = 1.0 / math.sqrt(D)
    q = torch.randn(B, H, 1, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16)
    query_pos = 3 * L
    tp = torch.zeros(B, G, C, device=DEV, dtype=torch.int32)
    for b in range(B):
        for g in range(G):
            tp[b, g, :L] = torch.randperm(query_pos, device=DEV)[:L].to(torch.int32)
    slot = torch.randint(0, L, (B, G), device=DEV, dtype=torch.int32)
    tp.scatter_(2, slot.long().unsqueeze(-1), torch.full((B, G, 1), query_pos, device=DEV, dtype=torch.int32))  # the query's own token
    kw = dict(softcap=softcap, sliding_window=window, token_pos=tp, query_pos=query_pos)
    if bits == 16:
        out, w = _cuda().decode_attention(q, k, v, scale, L, True, **kw)
        k_eff, v_eff = k[:, :, :L], v[:, :, :L]
    else:
        qk, sk, zk = ref.quantize_rows(k, bits)
        qv, sv, zv = ref.quantize_rows(v, bits)
        k_new = torch.randn(B, G, D, device=DEV, dtype=torch.bfloat16)
        v_new = torch.randn(B, G, D, device=DEV, dtype=torch.bfloat16)
        out, w = _cuda().decode_attention(q, qk, qv, scale, L, True, quant=(sk, zk, sv, zv, bits), new_kv=(k_new, v_new, slot), **kw)
        k_eff = ref.dequantize_rows(qk, sk, zk, bits, torch.bfloat16)[:, :, :L].clone()
        v_eff = ref.dequantize_rows(qv, sv, zv, bits, torch.bfloat16)[:, :, :L].clone()
        idx = slot.long().view(B, G, 1, 1).expand(B, G, 1, D)
        k_eff.scatter_(2, idx, k_new.unsqueeze(2))
        v_eff.scatter_(2, idx, v_new.unsqueeze(2))
    out_r, w_r = ref.sdpa(q, k_eff, v_eff, scale, query_pos, tp[:, :, :L], True, window, softcap)
    torch.testing.assert_close(out.float(), out_r.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(w, w_r, atol=1e-3, rtol=2e-2)
    if window is not None:
        assert bool((w[tp[:, :, :L] <= query_pos - window] == 0).all())


@pytest.mark.parametrize("dim,rows", [(1024, 777), (2560, 777), (3072, 777), (4096, 4), (2560, 1), (5120, 64)])
def test_add_rmsnorm_fused(dim, rows):
    """s = x + res; y = rmsnorm(s): one kernel forward, one kernel backward (with the gradient of
    the residual path added in the same pass), against the fp32 restatement."""
    from keys_values_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(rows, dim, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, dim, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(dim, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    y, s = ops.add_rmsnorm(x, r, w, 1e-6, False)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    (y.float() * gy.float()).sum().backward(retain_graph=True)
    gx1 = x.grad.clone()
    x.grad = None
    r.grad = None
    ((y.float() * gy.float()).sum() + (s.float() * gs.float()).sum()).backward()
    # reference in fp32 from the bf16-rounded sum
    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True)
    sf = (xf + rf).to(torch.bfloat16).float() + 0 * (xf + rf)  # value of the rounded sum, gradient of the sum
    yf = ref.rmsnorm(sf, w.float(), 1e-6, False)
    ((yf * gy.float()).sum() + (sf * gs.float()).sum()).backward()
    assert torch.equal(s.detach(), (x.detach().float() + r.detach().float()).to(torch.bfloat16))
    assert _rel_err(y.detach(), yf.detach()) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 2e-2
    assert _rel_err(r.grad, rf.grad) < 2e-2
    assert gx1.isfinite().all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [1000, 151936, 32003])
def test_ce_loss_kernels(dtype, V):
    from keys_values_b200 import ops

    torch.manual_seed(1)
    N = 37
    logits = (torch.randn(N, V, device=DEV) * 3).to(dtype).requires_grad_(True)
    targets = torch.randint(0, V, (N,), device=DEV)
    targets[3] = -100
    loss = ops.cross_entropy_rows(logits, targets, -100)
    g = torch.rand(N, device=DEV)
    (loss * g).sum().backward()
    lf = logits.detach().float().requires_grad_(True)
    ref_loss = torch.nn.functional.cross_entropy(lf, targets, ignore_index=-100, reduction="none")
    (ref_loss * g).sum().backward()
    torch.testing.assert_close(loss, ref_loss, atol=2e-3, rtol=1e-4)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel_err(logits.grad, lf.grad) < tol
    assert loss[3] == 0 and logits.grad[3].abs().max() == 0


def test_verification_api_and_host_optimizer_on_gpu():
    """The user-facing equivalence check (kernels against the fp32 restatement) and the host-resident
    optimizer with pinned staging on a GPU."""
    from keys_values_b200.attention.verification import verify_backend_equivalence, verify_backend_equivalence_batch
    from keys_values_b200.optimize.host_optimizer import HostOffloadOptimizer

    D = 128
    scale = 1.0 / math.sqrt(D)
    mk = lambda *s: torch.randn(*s, device=DEV, dtype=torch.bfloat16)  # noqa: E731
    cases = [
        dict(query=mk(1, 8, 64, D), key=mk(1, 2, 512, D), value=mk(1, 2, 512, D), scale_factor=scale, input_pos=448, return_attn_weights=True),
        dict(query=mk(2, 8, 1, D), key=mk(2, 2, 300, D), value=mk(2, 2, 300, D), scale_factor=scale, input_pos=299, return_attn_weights=True),
    ]
    passed, failed, results = verify_backend_equivalence_batch(cases, log_results=False)
    assert (passed, failed) == (2, 0) and all(r.weights_max_diff is not None for r in results)
    bad = verify_backend_equivalence(**cases[0], rtol=0.0, atol=0.0, log_results=False)
    assert not bad and bad.output_max_diff > 0
    w = torch.nn.Parameter(torch.ones(1000, device=DEV, dtype=torch.bfloat16))
    opt = HostOffloadOptimizer([w], lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.0))
    assert opt.host_params[0].is_pinned()
    for _ in range(3):
        opt.zero_grad()
        w.grad = torch.ones_like(w)
        opt.step()
    torch.cuda.synchronize()
    assert abs(float(w.detach()[0]) - 0.97) < 5e-3 and abs(float(opt.host_params[0].detach()[0]) - 0.97) < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("R,V", [(4, 128256), (1, 1000), (7, 33)])
def test_argmax_rows(dtype, R, V):
    from keys_values_b200 import ops

    x = torch.randn(R, V + 5, device=DEV, dtype=dtype)[:, :V]  # rows with a stride
    x[0, V // 2] = 100.0
    if V > 40 and R > 1:
        x[-1, 17] = x[-1, 40] = 50.0  # equal maxima: the first one counts
    for _ in range(2):  # the counters of the work space return to zero
        got = ops.argmax_rows(x)
        assert got.dtype == torch.int64 and got.shape == (R,)
        assert bool(((got >= 0) & (got < V)).all())  # checked before anything indexes with it
        assert torch.equal(x.gather(1, got.view(-1, 1)).view(-1), x.max(dim=-1).values)
        assert int(got[0]) == V // 2
        if V > 40 and R > 1:
            assert int(got[-1]) == 17
