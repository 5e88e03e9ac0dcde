"""Chunk/cell scheduling, chunked loss, gradients through the cache, generation, heads."""
import pytest
import torch

from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel, NaiveGPTAndHeadModel
from keys_values_b200.long_context import LongContextInferenceModel, create_chunk_sizes, get_chunk_of_targets, get_chunks_for_cells
from keys_values_b200.models import lora as lora_mod
from keys_values_b200.models.head_model import CrossEntropyOnLogits, HeadModelFactory, SequenceClassification, SequenceClassificationOnLogits
from keys_values_b200.models.model import GPT


def _lora_model(seed=0, **kw):
    torch.manual_seed(seed)
    cfg = lora_mod.Config.from_name("tiny-gpt", lora_r=4, lora_alpha=8, lora_query=True, lora_key=True, lora_value=True, lora_projection=True, **kw)
    m = lora_mod.GPT(cfg)
    m.apply(m._init_weights)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(m)
    return cfg, m


def _grads(m):
    g = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    m.zero_grad()
    return g


def test_chunk_and_cell_schedule():
    _, m = _lora_model()
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 1, 64, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=16)))
    assert create_chunk_sizes(m, 200, 16) == [64] + [16] * 8 + [8]
    assert create_chunk_sizes(m, 50, 16) == [50]
    cells = get_chunks_for_cells([64, 16, 16, 16, 16, 8], 40)
    assert [c.chunk_sizes for c in cells] == [(64,), (16, 16), (16, 16, 8)]
    assert [(c.start, c.end) for c in cells] == [(0, 64), (64, 96), (96, 136)]
    t = torch.arange(10).view(1, 10)
    assert get_chunk_of_targets(t, 0, 90, 100) is None
    assert get_chunk_of_targets(t, 88, 96, 100).tolist() == [[0, 1, 2, 3, 4, 5]]
    torch.manual_seed(0)
    sizes = create_chunk_sizes(m, 400, 16, randomize_chunk_sizes=True)
    assert sum(sizes) == 400 and sizes[0] == 64 and all(8 <= s <= 24 for s in sizes[1:-1])


def test_chunked_dense_loss_equals_plain_forward():
    _, m = _lora_model()
    head = CrossEntropyOnLogits(m.config)
    ids, tg = torch.randint(0, 512, (2, 150)), torch.randint(0, 512, (2, 40))
    m.assign_kv_caches(KVCacheFactory.create(m, "dense-default", 2, 160, dtype=torch.float32))
    # dense cache of 160 slots: prefill covers everything; force chunks with a smaller prefill via lastrec of equal length
    lcm = LongContextInferenceModel(m, head, chunk_size=16)
    loss = lcm(ids, tg)
    with torch.no_grad():
        want = NaiveGPTAndHeadModel(m, head)(ids, tg)
    torch.testing.assert_close(loss.mean(), want, atol=1e-5, rtol=1e-5)
    # logits of the last position without targets
    logits = lcm(ids, None)
    m.clear_kv_caches()
    with torch.no_grad():
        full = m(ids)
    torch.testing.assert_close(logits[:, 0], full[:, -1], atol=1e-4, rtol=1e-4)


def test_gradients_dense_chunked_equal_naive():
    _, m = _lora_model()
    head = CrossEntropyOnLogits(m.config)
    ids, tg = torch.randint(0, 512, (2, 120)), torch.randint(0, 512, (2, 30))
    m.assign_kv_caches(KVCacheFactory.create(m, "dense-default", 2, 128, dtype=torch.float32))
    gm = LongContextGradientModel(m, head, layers_per_cell=1, chunk_size=16)
    gm.train()
    loss = gm(ids, tg)
    loss.backward()
    g1 = _grads(m)
    l2 = NaiveGPTAndHeadModel(m, head)(ids, tg)
    l2.backward()
    g2 = _grads(m)
    torch.testing.assert_close(loss.value, l2.detach(), atol=1e-6, rtol=1e-6)
    assert g1.keys() == g2.keys() and len(g1) > 0
    for k in g1:
        torch.testing.assert_close(g1[k], g2[k], atol=2e-5, rtol=4e-5)


@pytest.mark.parametrize("name", ["h2o-default", "lastrec-default", "h2o-vlen-default"])
@pytest.mark.parametrize("lpc", [1, 2])
def test_gradients_multi_cell_equal_single_cell(name, lpc):
    _, m = _lora_model()
    head = CrossEntropyOnLogits(m.config)
    ids, tg = torch.randint(0, 512, (2, 200)), torch.randint(0, 512, (2, 64))
    ck = dict(max_chunk_size=16) if "h2o" in name else None
    m.assign_kv_caches(KVCacheFactory.create(m, name, 2, 64, dtype=torch.float32, cache_kwargs=ck))
    res = []
    for mult, layers in ((1.0, lpc), (100.0, 2)):
        gm = LongContextGradientModel(m, head, layers_per_cell=layers, chunk_size=16, chunks_per_cell_multiplier=mult)
        gm.train()
        loss = gm(ids, tg)
        n_cells = len(gm.cells)
        loss.backward()
        res.append((loss.item(), _grads(m), n_cells))
    assert res[0][2] > 2 and res[1][2] == 1
    assert abs(res[0][0] - res[1][0]) < 1e-6
    for k in res[0][1]:
        torch.testing.assert_close(res[0][1][k], res[1][1][k], atol=2e-5, rtol=4e-5)
    # train mode and eval mode give the same loss
    gm.eval()
    torch.testing.assert_close(gm(ids, tg).mean(), torch.tensor(res[0][0]), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("name", ["tiny-gemma2", "tiny-llama-d64", "tiny-gemma2-d256"])
def test_gradients_window_softcap_and_small_heads_chunked_equal_naive(name):
    """A Gemma-2 style model (one layer with a sliding window, capped attention scores and logits, post norms) and a model
    with head size 64: the chunked pass over a cache that holds the whole sequence equals whole-sequence autograd."""
    from keys_values_b200.config import Config

    torch.manual_seed(0)
    cfg = Config.from_name(name)
    m = GPT(cfg)
    m.apply(m._init_weights)
    head = CrossEntropyOnLogits(cfg)
    T, C, cs = 320, 384, 64  # the window of the Gemma-style layer (96) is shorter than the sequence
    ids = torch.randint(0, cfg.vocab_size, (1, T))
    tg = torch.randint(0, cfg.vocab_size, (1, 64))
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 1, C, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=cs)))
    gm = LongContextGradientModel(m, head, layers_per_cell=1, chunk_size=cs)
    gm.train()
    loss = gm(ids, tg)
    loss.backward()
    g1 = _grads(m)
    l2 = NaiveGPTAndHeadModel(m, head)(ids, tg)
    l2.backward()
    g2 = _grads(m)
    assert abs(float(loss.value) - float(l2.detach())) < 1e-4
    assert g1.keys() == g2.keys() and len(g1) > 0
    for k in g1:
        torch.testing.assert_close(g1[k], g2[k], atol=2e-5, rtol=1e-3)


def test_gradients_quantized_cache_and_saved_attention():
    _, m = _lora_model()
    head = CrossEntropyOnLogits(m.config)
    ids, tg = torch.randint(0, 512, (1, 200)), torch.randint(0, 512, (1, 64))
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-torch-quantized8", 1, 64, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=16)))
    res = []
    for save, offload, qn in ((False, False, None), (True, False, None), (False, True, "torch-quantized8")):
        gm = LongContextGradientModel(m, head, layers_per_cell=1, chunk_size=16, save_attention_outputs=save, offload_checkpoints=offload,
                                      layercp_qname=qn)
        gm.train()
        loss = gm(ids, tg)
        loss.backward()
        res.append((loss.item(), _grads(m)))
    for k in res[0][1]:
        torch.testing.assert_close(res[0][1][k], res[1][1][k], atol=1e-7, rtol=1e-6)
        # int8 layer-input checkpoints perturb the gradients slightly
        assert (res[0][1][k] - res[2][1][k]).norm() <= 0.05 * res[0][1][k].norm() + 1e-6


def test_full_finetune_embedding_gradient():
    torch.manual_seed(0)
    m = GPT.from_name("tiny-gpt")
    m.apply(m._init_weights)
    head = CrossEntropyOnLogits(m.config)
    ids, tg = torch.randint(0, 512, (1, 100)), torch.randint(0, 512, (1, 20))
    m.assign_kv_caches(KVCacheFactory.create(m, "dense-default", 1, 128, dtype=torch.float32))
    gm = LongContextGradientModel(m, head, layers_per_cell=2, chunk_size=16)
    gm.train()
    gm(ids, tg).backward()
    g1 = _grads(m)
    NaiveGPTAndHeadModel(m, head)(ids, tg).backward()
    g2 = _grads(m)
    for k in g2:
        torch.testing.assert_close(g1[k], g2[k], atol=3e-5, rtol=1e-4)


def test_heads():
    cfg, m = _lora_model()
    assert HeadModelFactory.is_supported("next_token_prediction")
    h = SequenceClassificationOnLogits(cfg, [3, 7, 9])
    logits = torch.randn(2, 5, cfg.padded_vocab_size)
    loss = h(logits, torch.tensor([[0], [2]]), 0)
    want = torch.nn.functional.cross_entropy(logits[:, -1, [3, 7, 9]], torch.tensor([0, 2]), reduction="none")
    torch.testing.assert_close(loss, want)
    h2 = SequenceClassification(cfg, num_classes=3, pool_type="mean")
    x = torch.randn(2, 8, cfg.n_embd)
    assert h2(x[:, :5], None, 0) == 0
    out = h2(x[:, 5:], torch.tensor([[1], [0]]), 5)
    want = torch.nn.functional.cross_entropy(h2.linear_head(x.mean(1)), torch.tensor([1, 0]), reduction="none")
    torch.testing.assert_close(out, want, atol=1e-6, rtol=1e-5)


def test_generation_batched_equals_single_and_stops():
    from keys_values_b200.generate.base import batched_generate_fn, generate

    torch.manual_seed(0)
    m = GPT.from_name("tiny-gpt")
    m.apply(m._init_weights)
    m.eval()
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 2, 64, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=16)))
    p1, p2 = torch.randint(0, 512, (90,)), torch.randint(0, 512, (90,))
    s1 = generate(m, p1, 100, prompt_chunksize=16, temperature=0.0, include_prompt=False)
    s2 = generate(m, p2, 100, prompt_chunksize=16, temperature=0.0, include_prompt=False)
    rows = [[], []]
    for toks in batched_generate_fn(m, torch.stack([p1, p2]), 100, 16, dict(temperature=0.0), include_prompt=False):
        for b, t in enumerate(toks):
            if t is not None:
                rows[b].append(int(t))
    assert rows[0] == s1.tolist() and rows[1] == s2.tolist()
    stop = ([rows[0][2]],)
    got = [int(t[0]) for t in batched_generate_fn(m, p1.view(1, -1), 100, 16, dict(temperature=0.0), stop, include_prompt=False) if t[0] is not None]
    assert got == rows[0][:3]


def test_lora_merge_and_state_dict_compat():
    cfg, m = _lora_model()
    base_sd = {k.replace(".linear.", "."): v for k, v in m.state_dict().items() if "lora_" not in k}
    _, m2 = _lora_model(seed=1)
    missing = m2.load_state_dict(base_sd, strict=False)
    assert all("lora_" in k for k in missing.missing_keys) and not missing.unexpected_keys
    x = torch.randint(0, 512, (1, 20))
    with torch.no_grad():
        before = m(x)
        lora_mod.merge_lora_weights(m)
        after = m(x)
    torch.testing.assert_close(before, after, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("enable", [(True, False, True), (False, True, False), (True, True, True)])
def test_lora_qkv_parts_forward_and_gradients_match_the_definition(enable):
    """The fused form (sum and scaling in the epilogue of the low-rank product, one block matrix for the enabled parts)
    against the definition: linear(x) + scaling · x (B A)^T with the update of disabled parts zero; gradients too."""
    torch.manual_seed(0)
    lin = lora_mod.LoRAQKVLinear(48, head_size=8, n_head=4, n_query_groups=2, r=4, lora_alpha=8, enable_lora=enable, bias=True)
    torch.nn.init.normal_(lin.lora_B, std=0.2)
    x = torch.randn(2, 7, 48, requires_grad=True)
    y = lin(x)
    y.square().sum().backward()
    got = (y.detach().clone(), x.grad.clone(), lin.lora_A.grad.clone(), lin.lora_B.grad.clone())
    x.grad = lin.lora_A.grad = lin.lora_B.grad = None
    y_def = torch.nn.functional.linear(x, lin.linear.weight + lin.get_lora_AB(), lin.linear.bias)
    y_def.square().sum().backward()
    want = (y_def.detach(), x.grad, lin.lora_A.grad, lin.lora_B.grad)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-4)
    # the outputs of a disabled part are those of the frozen linear alone
    base = torch.nn.functional.linear(x, lin.linear.weight, lin.linear.bias)
    off = 0
    for size, on in zip((32, 16, 16), enable):
        if not on:
            torch.testing.assert_close(y[..., off:off + size], base[..., off:off + size])
        off += size


def test_dora_forward_matches_definition():
    torch.manual_seed(0)
    lin = lora_mod.DoRALinear(16, 12, r=4, lora_alpha=8)
    torch.nn.init.normal_(lin.lora_B, std=0.1)
    x = torch.randn(3, 16)
    w = lin.linear.weight + lin.get_lora_AB()
    want = torch.nn.functional.linear(x, w * (lin.lora_scales / w.norm(dim=1)).unsqueeze(-1), lin.linear.bias)
    torch.testing.assert_close(lin(x), want, atol=1e-5, rtol=1e-5)
    y0 = lin(x)
    lin.merge()
    torch.testing.assert_close(lin(x), y0, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("chunk", [8, 24])
def test_gradients_with_grace_period(chunk, monkeypatch):
    """Score-based cache with a grace ring (the newest tokens cannot be evicted): the replay moves the
    oldest ring entries to the evicted slots as the forward pass did. Multi-cell equals single-cell, the
    training pass equals the inference pass, and the gradient agrees with finite differences in fp64."""
    import keys_values_b200.kvcache.h2o as h2o_mod

    # The slots to evict are chosen by age instead of by score, so that the decisions do not depend on
    # the weights and finite differences are a valid oracle (the gradient treats decisions as constants).
    def oldest_first(scores, weights, k_select, n_evictable, normalize=False, token_pos=None, input_pos=0, prefill_length=0, out=None):
        if weights is not None:
            scores += weights
        return torch.argsort(token_pos[:, :, :n_evictable], dim=-1)[:, :, :k_select].to(torch.int32)

    monkeypatch.setattr(h2o_mod.ops, "h2o_update", oldest_first)
    torch.manual_seed(0)
    cfg = lora_mod.Config.from_name("tiny-gpt", lora_r=4, lora_alpha=8, lora_query=True, lora_value=True)
    m = lora_mod.GPT(cfg)
    m.apply(m._init_weights)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(m)
    m = m.double()
    head = CrossEntropyOnLogits(cfg)
    ids, tg = torch.randint(0, 512, (2, 150)), torch.randint(0, 512, (2, 40))
    kw = dict(max_chunk_size=chunk, grace_period=12)  # chunks shorter and longer than the ring
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 2, 48, dtype=torch.float64, cache_kwargs=kw))
    res = []
    for mult, layers in ((1.0, 1), (100.0, 2)):
        gm = LongContextGradientModel(m, head, layers_per_cell=layers, chunk_size=chunk, chunks_per_cell_multiplier=mult)
        gm.train()
        loss = gm(ids, tg)
        loss.backward()
        res.append((loss.item(), _grads(m), len(gm.cells)))
    assert res[0][2] > 2 and res[1][2] == 1 and abs(res[0][0] - res[1][0]) < 1e-9
    for k in res[0][1]:
        torch.testing.assert_close(res[0][1][k], res[1][1][k], atol=1e-9, rtol=1e-7)
    gm.eval()
    with torch.no_grad():
        assert abs(float(gm(ids, tg).mean()) - res[0][0]) < 1e-9
    # central differences along a random direction in two parameters (the slot decisions are not differentiated)
    names = [n for n in res[0][1] if "lora_B" in n][:2]
    params = dict(m.named_parameters())
    for n in names:
        d = torch.randn_like(params[n])
        eps = 1e-3  # the loss comes back in fp32
        vals = []
        for sgn in (1.0, -1.0):
            with torch.no_grad():
                params[n].add_(sgn * eps * d)
                vals.append(float(gm(ids, tg).mean()))
                params[n].sub_(sgn * eps * d)
        fd = (vals[0] - vals[1]) / (2 * eps)
        an = float((res[0][1][n] * d).sum())
        assert abs(fd - an) <= 5e-3 * abs(an) + 2e-4, (n, fd, an)


def test_profile_parts_reports_forward_and_backward(capsys):
    """``profile_parts``: a cProfile report per part of the step, the step itself unchanged."""
    from keys_values_b200.config import Config
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
    from keys_values_b200.models.head_model import CrossEntropyOnLogits
    from keys_values_b200.models.model import GPT

    torch.manual_seed(0)
    cfg = Config.from_name("tiny-gpt")
    losses = []
    for parts in (None, "both"):
        torch.manual_seed(1)
        gpt = GPT(cfg)
        gpt.apply(gpt._init_weights)
        gpt.assign_kv_caches(KVCacheFactory.create(gpt, "lastrec-default", 1, 48, dtype=torch.float32))
        gm = LongContextGradientModel(gpt, CrossEntropyOnLogits(cfg), layers_per_cell=1, chunk_size=16, profile_parts=parts)
        gm.train()
        ids, tg = torch.arange(96).view(1, 96) % cfg.vocab_size, torch.arange(16).view(1, 16)
        loss = gm(ids, tg)
        loss.backward()
        losses.append(float(loss))
        if parts:
            assert set(gm.part_profiler.reports) == {"forward", "backward"}
            assert "cumulative" in gm.part_profiler.reports["backward"]
    assert losses[0] == losses[1]
    assert "cProfile of the forward part" in capsys.readouterr().out
    with pytest.raises(ValueError):
        LongContextGradientModel(gpt, CrossEntropyOnLogits(cfg), layers_per_cell=1, chunk_size=16, profile_parts="sideways")
