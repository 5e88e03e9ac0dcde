"""Guard zones around every buffer that a kernel writes into: a stand-in for a memory checker. Each buffer is
the middle of a larger allocation whose head and tail hold a bit pattern; after the kernel ran on odd shapes
(ragged last tiles, sizes that are no multiple of a tile) the pattern must be intact, and a second run of the
same call must give the same bits."""
import math

import pytest
import torch

from keys_values_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
GUARD = 4096  # bytes on either side


class Guarded:
    def __init__(self):
        self.zones = []

    def like(self, t: torch.Tensor) -> torch.Tensor:
        """A copy of ``t`` that lives between two guard zones."""
        nbytes = t.numel() * t.element_size()
        pad = (-nbytes) % 256
        raw = torch.empty(GUARD + nbytes + pad + GUARD, dtype=torch.uint8, device=t.device)
        raw.fill_(0xA5)
        mid = raw[GUARD : GUARD + nbytes].view(t.dtype).view(t.shape)
        mid.copy_(t)
        self.zones.append((raw, nbytes))
        return mid

    def check(self):
        torch.cuda.synchronize()
        for raw, nbytes in self.zones:
            assert bool((raw[:GUARD] == 0xA5).all()), "a kernel wrote in front of its buffer"
            assert bool((raw[GUARD + nbytes :] == 0xA5).all()), "a kernel wrote behind its buffer"


def _cuda():
    from keys_values_b200.ops import cuda

    return cuda


def test_attention_backward_stays_inside_its_gradient_buffers():
    B, H, G, T, L, D = 1, 8, 2, 77, 333, 128
    g = Guarded()
    q = torch.randn(B, H, T, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, G, L, D, device=DEV, dtype=torch.bfloat16)
    go = torch.randn(B, T, H * D, device=DEV, dtype=torch.bfloat16)
    tp = torch.stack([torch.randperm(L, device=DEV) for _ in range(B * G)]).view(B, G, L).to(torch.int32)
    new = torch.randperm(L, device=DEV)[:T]
    tp[:, :, new] = (torch.arange(T, device=DEV) + 2 * L).to(torch.int32)
    scale = 1 / math.sqrt(D)
    out, w, lse = _cuda().sdpa_fwd(q, k, v, scale, 2 * L, tp, True)
    results = []
    for _ in range(2):
        dk, dv = g.like(torch.zeros(B, G, L, D, device=DEV)), g.like(torch.zeros(B, G, L, D, device=DEV))
        dq, _, _ = _cuda().sdpa_bwd(go, q, k, v, out, lse, scale, 2 * L, tp, dk, dv)
        results.append((dq.clone(), dk.clone(), dv.clone()))
    g.check()
    _cuda().check_status(DEV)
    for a, b in zip(*results):
        assert torch.equal(a, b)  # run to run identical


@pytest.mark.parametrize("bits", [0, 8, 4])
def test_cache_write_stays_inside_the_cache(bits):
    B, G, C, D, n = 2, 3, 37, 128, 5
    g = Guarded()
    kb = g.like(torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16))
    vb = g.like(torch.randn(B, G, C, D, device=DEV, dtype=torch.bfloat16))
    tp = g.like(torch.zeros(B, G, C, device=DEV, dtype=torch.int32))
    slots = torch.stack([torch.randperm(C, device=DEV)[:n] for _ in range(B * G)]).view(B, G, n).to(torch.int32)
    slots[:, :, -1] = C - 1  # the very last row of the buffers
    key, val = torch.randn(B, G, n, D, device=DEV, dtype=torch.bfloat16), torch.randn(B, G, n, D, device=DEV, dtype=torch.bfloat16)
    if bits == 0:
        ops.cache_write(kb, vb, tp, slots, key, val, 100)
    else:
        Dq = D if bits == 8 else D // 2
        qk, qv = g.like(torch.zeros(B, G, C, Dq, device=DEV, dtype=torch.uint8)), g.like(torch.zeros(B, G, C, Dq, device=DEV, dtype=torch.uint8))
        sk, sv = g.like(torch.ones(B, G, C, device=DEV)), g.like(torch.ones(B, G, C, device=DEV))
        zk, zv = g.like(torch.zeros(B, G, C, device=DEV, dtype=torch.int32)), g.like(torch.zeros(B, G, C, device=DEV, dtype=torch.int32))
        ops.cache_write_quant(kb, vb, tp, slots, key, val, 100, qk, sk, zk, qv, sv, zv, bits)
    g.check()
    _cuda().check_status(DEV)


def test_score_update_and_selection_stay_inside_the_score_buffer():
    B, G, C, k = 2, 3, 1001, 37
    g = Guarded()
    start = torch.rand(B, G, C, device=DEV)
    scores = g.like(start)
    w = torch.rand(B, G, C, device=DEV)
    tp = torch.stack([torch.randperm(C, device=DEV) for _ in range(B * G)]).view(B, G, C).to(torch.int32)
    first = ops.h2o_update(scores, w, k, C - 3, True, tp, C + 5, 17).clone()
    g.check()
    scores2 = g.like(start)  # the same state again
    again = ops.h2o_update(scores2, w, k, C - 3, True, tp, C + 5, 17)
    g.check()
    assert torch.equal(first, again)  # the same evictions, in the same order
    _cuda().check_status(DEV)
