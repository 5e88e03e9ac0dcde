"""KV-cache policies and buffers against brute-force restatements (CPU, fp32)."""
import math

import pytest
import torch

from keys_values_b200.kvcache.factory import KVCacheFactory, SUPPORTED_CACHES
from keys_values_b200.kvcache.utils import smallest_covering_ranges
from keys_values_b200.models.model import GPT
from keys_values_b200.ops import reference as ref


def _model(name="tiny-gpt"):
    torch.manual_seed(0)
    m = GPT.from_name(name)
    m.apply(m._init_weights)
    return m.eval()


def test_supported_names():
    names = KVCacheFactory.supported_names()
    assert "h2o-torch-quantized8" in names and "dense-default" in names and "qh2o-default" not in names
    with pytest.raises(ValueError):
        KVCacheFactory._cache_type("qh2o-default")


@pytest.mark.parametrize("name", ["dense-default", "dense-torch-quantized8"])
def test_dense_cache_equals_no_cache(name):
    m = _model()
    idx = torch.randint(0, 512, (2, 96))
    with torch.no_grad():
        want = m(idx)
        m.assign_kv_caches(KVCacheFactory.create(m, name, 2, 128, dtype=torch.float32))
        m.reset()
        outs = [m(idx[:, :40])] + [m(idx[:, s : s + 8]) for s in range(40, 96, 8)]
    got = torch.cat(outs, 1)
    tol = 1e-5 if name.endswith("default") else 5e-2
    torch.testing.assert_close(got, want, atol=tol, rtol=tol)


def test_dense_cache_full_raises():
    m = _model()
    m.assign_kv_caches(KVCacheFactory.create(m, "dense-default", 1, 16, dtype=torch.float32))
    m.reset()
    with torch.no_grad():
        m(torch.randint(0, 512, (1, 16)))
        with pytest.raises((IndexError, ValueError)):
            m(torch.randint(0, 512, (1, 1)))


def test_lastrec_ring_keeps_sinks_and_recent():
    m = _model()
    C = 32
    caches = KVCacheFactory.create(m, "lastrec-default", 1, C, dtype=torch.float32, cache_kwargs=dict(init_grace_tokens=4))
    m.assign_kv_caches(caches)
    m.reset()
    with torch.no_grad():
        m(torch.randint(0, 512, (1, C)))
        for s in range(5):
            m(torch.randint(0, 512, (1, 7)))
    tp = caches[0].token_positions()[0, 0].tolist()
    total = C + 35
    assert sorted(tp[:4]) == [0, 1, 2, 3]
    assert sorted(tp[4:]) == list(range(total - (C - 4), total))


def test_h2o_scores_match_brute_force_and_evict_lowest():
    torch.manual_seed(1)
    m = _model()
    C, chunk = 32, 4
    caches = KVCacheFactory.create(m, "h2o-default", 2, C, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=chunk, keep_initial_fraction=0.0))
    m.assign_kv_caches(caches)
    m.reset()
    idx = torch.randint(0, 512, (2, C + 3 * chunk))
    with torch.no_grad():
        m(idx[:, :C])
        m(idx[:, C : C + chunk])  # initial rule: overwrites slots [0, chunk)
        c0 = caches[0]
        scores_before = c0.scores[:2].clone()
        nxt = c0.next_positions(chunk).clone()
        # the next slots are the `chunk` lowest scores
        want = torch.topk(scores_before, chunk, dim=-1, largest=False)[1]
        assert torch.equal(nxt.sort(-1)[0].long(), want.sort(-1)[0])
        m(idx[:, C + chunk : C + 2 * chunk])
    tp = c0.token_positions()
    # the tokens just written sit in the chosen slots
    got = tp.gather(2, nxt.long()).sort(-1)[0]
    assert torch.equal(got, torch.arange(C + chunk, C + 2 * chunk, dtype=torch.int32).expand_as(got))


def test_h2o_grace_period_never_evicts_recent_tokens():
    m = _model()
    C, g, chunk = 32, 8, 4
    caches = KVCacheFactory.create(m, "h2o-default", 1, C, dtype=torch.float32, cache_kwargs=dict(grace_period=g, max_chunk_size=chunk))
    m.assign_kv_caches(caches)
    m.reset()
    total = C
    with torch.no_grad():
        m(torch.randint(0, 512, (1, C)))
        for _ in range(6):
            m(torch.randint(0, 512, (1, chunk)))
            total += chunk
            for c in caches:
                tp = c.token_positions()[0]
                for row in tp:
                    present = set(row.tolist())
                    assert all(t in present for t in range(total - g, total)), "a token inside the grace period was evicted"
                    assert len(present) == C


@pytest.mark.parametrize("bits", [8, 4])
def test_quantization_roundtrip_error_bound(bits):
    x = torch.randn(3, 2, 17, 64)
    q, s, z = ref.quantize_rows(x, bits)
    d = ref.dequantize_rows(q, s, z, bits, torch.float32)
    assert q.shape[-1] == (64 if bits == 8 else 32)
    assert ((d - x).abs() <= 0.5001 * s.unsqueeze(-1) + 1e-6).all()


def test_quantized_buffers_share_scratch_and_requantize_once_per_visit():
    m = _model()
    caches = KVCacheFactory.create(m, "h2o-torch-quantized8", 1, 32, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=4))
    assert caches[0].kv_buffers.dequant_buffers is caches[1].kv_buffers.dequant_buffers
    m.assign_kv_caches(caches)
    m.reset()
    with torch.no_grad():
        m(torch.randint(0, 512, (1, 32)))
        n0 = caches[0].kv_buffers.dequant_buffers.num_dequantizations
        m(torch.randint(0, 512, (1, 4)), chunk_sizes=None)
    # two layers alternate on the scratch: one de-quantization per (call, layer)
    assert caches[0].kv_buffers.dequant_buffers.num_dequantizations - n0 == 2
    total, parts = KVCacheFactory.size_estimate(caches)
    assert total > 0 and "dequant_buffers" in parts


def test_offloader_matches_plain_quantized():
    m = _model()
    idx = torch.randint(0, 512, (1, 64))
    outs = []
    for offload in (False, True):
        if offload:
            caches, off = KVCacheFactory.create_cpu_offloading(m, "h2o-torch-quantized8", 1, 32, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=8), pin_memory=False)
        else:
            caches = KVCacheFactory.create(m, "h2o-torch-quantized8", 1, 32, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=8))
        m.assign_kv_caches(caches)
        m.reset()
        with torch.no_grad():
            o = [m(idx[:, :32])] + [m(idx[:, s : s + 8]) for s in range(32, 64, 8)]
        outs.append(torch.cat(o, 1))
    torch.testing.assert_close(outs[0], outs[1])


def test_size_estimate_matches_apriori():
    m = _model()
    for name in ("h2o-default", "lastrec-default", "dense-default"):
        caches = KVCacheFactory.create(m, name, 2, 64, dtype=torch.float32)
        for c in caches:
            c.kv_buffers.allocate("cpu", torch.float32)
        total, _ = KVCacheFactory.size_estimate(caches)
        apriori, _ = KVCacheFactory.size_estimate_apriori(name, m.config, 2, 64, dtype=torch.float32)
        assert total == apriori


def test_smallest_covering_ranges():
    assert smallest_covering_ranges([1, 2, 3, 10, 11, 30], 2) == [(1, 12), (30, 31)]
    assert smallest_covering_ranges([], 3) == []
    assert smallest_covering_ranges([5], 1) == [(5, 6)]


def test_sdpa_weights_are_sum_over_queries_mean_over_group():
    B, H, G, T, L, D = 2, 4, 2, 5, 12, 16
    q, k, v = torch.randn(B, H, T, D), torch.randn(B, G, L, D), torch.randn(B, G, L, D)
    tp = torch.stack([torch.stack([torch.randperm(L) for _ in range(G)]) for _ in range(B)]).int() + 20
    tp[:, :, :T] = torch.arange(40, 40 + T)
    out, w = ref.sdpa(q, k, v, 1 / math.sqrt(D), 40, tp, True)
    kk = k.repeat_interleave(H // G, 1)
    s = torch.einsum("bhqd,bhkd->bhqk", q, kk) / math.sqrt(D)
    mask = tp.repeat_interleave(H // G, 1).unsqueeze(2) <= (40 + torch.arange(T)).view(1, 1, T, 1)
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    want = p.view(B, G, H // G, T, L).sum(dim=(2, 3)) / (H // G)
    torch.testing.assert_close(w, want, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(w.sum(-1), torch.full((B, G), float(T)), atol=1e-4, rtol=1e-5)


def test_smart_lastrec_protects_initial_part():
    from keys_values_b200.kvcache.smart_lastrec import SmartInitialLastRecentlyInsertedKVCache

    class Tok:
        def decode(self, ids):
            return "".join(chr(97 + (i % 26)) for i in ids)

    m = _model()
    C = 32
    caches = KVCacheFactory.create(m, "smart-lastrec-default", 1, C, dtype=torch.float32,
                                   cache_kwargs=dict(tokenizer=Tok(), end_initial_regex="cde", max_initial_fraction=0.5))
    assert isinstance(caches[0], SmartInitialLastRecentlyInsertedKVCache)
    m.assign_kv_caches(caches)
    m.reset()
    ids = torch.arange(C).view(1, C) % 26  # text "abcdef…": the initial part ends after "cde" = 5 tokens
    with torch.no_grad():
        m(ids)
        for _ in range(4):
            m(torch.randint(0, 26, (1, 10)))
    assert caches[0].protected[0] == (0, 5)
    tp = caches[0].token_positions()[0, 0]
    assert tp[:5].tolist() == [0, 1, 2, 3, 4]
    assert tp.max().item() == C + 40 - 1


def test_before_after_snapshots_catch_a_changed_cache(tmp_path):
    """Freeze the calls of an H2O cache, replay them through an identical cache (passes) and through one whose
    score update was tampered with (fails at the first call where a different slot is evicted)."""
    from keys_values_b200.kvcache.test_utils import ForwardSnapshots

    C, chunk = 32, 4
    idx = torch.randint(0, 512, (2, C + 4 * chunk), generator=torch.Generator().manual_seed(3))
    mask = str(tmp_path / "call_{}.pt")

    def run(mode, tamper=False):
        torch.manual_seed(1)
        m = _model()
        caches = KVCacheFactory.create(m, "h2o-default", 2, C, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=chunk))
        m.assign_kv_caches(caches)
        m.reset()
        snap = ForwardSnapshots(caches[0], mask, num_steps=5)
        getattr(snap, mode)()
        if tamper:
            inner = caches[0]._update if hasattr(caches[0], "_update") else None
            assert inner is not None

            def noisy(*a, **k):
                out = inner(*a, **k)
                caches[0].scores.mul_(-1.0)  # evict the most attended tokens instead of the least
                return out

            caches[0]._update = noisy
        with torch.no_grad():
            m(idx[:, :C])
            for s in range(C, idx.shape[1], chunk):
                m(idx[:, s : s + chunk])
        snap.stop()
        return snap

    run("store")
    assert run("compare").compared == [0, 1, 2, 3, 4]
    with pytest.raises(AssertionError):
        run("compare", tamper=True)
