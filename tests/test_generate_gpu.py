"""Generation on the GPU: single-token steps replayed from one CUDA graph produce the tokens of the
eager steps; the device-resident position drives the cache write, the score ageing and RoPE."""
import pytest
import torch

from keys_values_b200.config import Config
from keys_values_b200.generate.base import batched_generate_fn
from keys_values_b200.generate.decode_graph import DecodeGraph, Decoder
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.long_context import LongContextInferenceModel
from keys_values_b200.models.head_model import CrossEntropyOnLogits
from keys_values_b200.models.model import GPT

pytestmark = pytest.mark.gpu


def _setup(cache_name, B, C, cache_kwargs=None, model="tiny-qwen3"):
    dev, dtype = torch.device("cuda", 0), torch.bfloat16
    torch.manual_seed(0)
    cfg = Config.from_name(model)
    m = GPT(cfg)
    m.apply(m._init_weights)
    m = m.to(device=dev, dtype=dtype).eval()
    kw = dict(max_chunk_size=64) if "h2o" in cache_name else {}
    kw.update(cache_kwargs or {})
    m.assign_kv_caches(KVCacheFactory.create(m, cache_name, B, C, dtype=dtype, device=dev, cache_kwargs=kw))
    return cfg, m, dev


def _prefill(m, prompts, total):
    m.reset()
    lcm = LongContextInferenceModel(m, CrossEntropyOnLogits(m.config), chunk_size=64)
    lcm.fixed_max_seq_length = total
    return lcm(prompts, None)


@pytest.mark.parametrize("cache_name,cache_kwargs", [
    ("h2o-default", None), ("h2o-torch-quantized8", None), ("h2o-torch-quantized4", None), ("h2o-default", dict(normalize_scores=True)),
    ("lastrec-default", None), ("lastrec-torch-quantized8", None),
])
def test_graph_decode_equals_eager(cache_name, cache_kwargs):
    B, C, T, steps = 2, 256, 600, 24
    cfg, m, dev = _setup(cache_name, B, C, cache_kwargs)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), device=dev)
    results = {}
    with torch.inference_mode():
        for use_graph in (False, True):
            logits = _prefill(m, prompts, T + steps + 1)
            tok = logits.argmax(-1).view(B, 1)
            dec = Decoder(m, B, use_graph=use_graph)
            toks, lgs = [], []
            for _ in range(steps):
                lg = dec(tok)
                tok = lg[:, -1].argmax(-1, keepdim=True)
                toks.append(tok.clone())
                lgs.append(lg.float().clone())
            if use_graph:
                assert dec.graph is not None, dec.reason
                assert dec.graph.steps == steps - dec.warmup
            results[use_graph] = (torch.cat(toks, 1), torch.stack(lgs), [c.input_pos for c in m.get_kv_caches()],
                                  [c.token_positions().clone() for c in m.get_kv_caches()])
    (t0, l0, p0, tp0), (t1, l1, p1, tp1) = results[False], results[True]
    assert p0 == p1 == [T + steps] * cfg.n_layer
    assert torch.equal(t0, t1)
    assert torch.allclose(l0, l1, atol=2e-2, rtol=2e-2)
    for a, b in zip(tp0, tp1):  # the slots chosen and the positions written there agree
        assert torch.equal(a, b)


@pytest.mark.parametrize("cache_name", ["h2o-default", "h2o-torch-quantized8", "lastrec-default"])
def test_graph_decode_with_sliding_window_and_softcap(cache_name, monkeypatch):
    """A Gemma-2 style model (a layer with a window shorter than the cache, capped scores): the decode kernel serves it
    (strict mode: no restatement), captured steps give the tokens of eager steps, and the first step agrees with the
    PyTorch restatement of the same attention."""
    from keys_values_b200 import ops

    monkeypatch.setenv("KVB200_STRICT_NATIVE", "1")
    B, C, T, steps = 2, 256, 600, 16
    cfg, m, dev = _setup(cache_name, B, C, model="tiny-gemma2")
    prompts = torch.randint(0, cfg.vocab_size, (B, T), device=dev)
    results = {}
    with torch.inference_mode():
        for use_graph in (False, True):
            logits = _prefill(m, prompts, T + steps + 1)
            tok = logits.argmax(-1).view(B, 1)
            dec = Decoder(m, B, use_graph=use_graph)
            toks, lgs = [], []
            for _ in range(steps):
                lg = dec(tok)
                tok = lg[:, -1].argmax(-1, keepdim=True)
                toks.append(tok.clone())
                lgs.append(lg.float().clone())
            if use_graph:
                assert dec.graph is not None, dec.reason
            results[use_graph] = (torch.cat(toks, 1), torch.stack(lgs))
        assert torch.equal(results[False][0], results[True][0])
        assert torch.allclose(results[False][1], results[True][1], atol=2e-2, rtol=2e-2)
        # the same first step through the restatement
        monkeypatch.setenv("KVB200_STRICT_NATIVE", "0")
        ops.set_native_attention(False)
        try:
            logits = _prefill(m, prompts, T + steps + 1)
            lg = m(logits.argmax(-1).view(B, 1))
        finally:
            ops.set_native_attention(True)
        assert torch.allclose(lg.float(), results[False][1][0], atol=8e-2, rtol=5e-2)


def test_inference_with_head_size_256_runs_on_the_native_forward(monkeypatch):
    """Head size 256 with a window layer and capped scores: chunked prefill and single-token steps are served by the
    head-size-256 forward kernels (strict mode: no restatement), and agree with the PyTorch restatement step by step."""
    from keys_values_b200 import ops

    monkeypatch.setenv("KVB200_STRICT_NATIVE", "1")
    B, C, T, steps = 2, 256, 600, 6
    cfg, m, dev = _setup("h2o-default", B, C, model="tiny-gemma2-d256")
    prompts = torch.randint(0, cfg.vocab_size, (B, T), device=dev)
    with torch.inference_mode():
        logits = _prefill(m, prompts, T + steps + 1)
        tok = logits.argmax(-1).view(B, 1)
        toks, lgs = [tok.clone()], []
        for _ in range(steps):
            lg = m(tok)
            tok = lg[:, -1].argmax(-1, keepdim=True)
            toks.append(tok.clone())
            lgs.append(lg.float().clone())
        monkeypatch.setenv("KVB200_STRICT_NATIVE", "0")
        ops.set_native_attention(False)
        try:
            logits_r = _prefill(m, prompts, T + steps + 1)
            lgs_r = [m(t).float().clone() for t in toks[:steps]]  # the same tokens fed to the restatement
        finally:
            ops.set_native_attention(True)
    assert torch.allclose(logits.float(), logits_r.float(), atol=8e-2, rtol=5e-2)
    for a, b in zip(lgs, lgs_r):
        assert torch.allclose(a, b, atol=8e-2, rtol=5e-2)


def test_graph_decode_conditions_and_generate_api():
    B, C, T = 2, 256, 100
    cfg, m, dev = _setup("h2o-default", B, C)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), device=dev)
    with torch.inference_mode():
        _prefill(m, prompts, 400)
        assert "not full" in DecodeGraph.why_not(m)  # 100 of 256 slots are in use
    # public API: same tokens with and without the graph (the prompt fills the cache)
    prompts = torch.randint(0, cfg.vocab_size, (B, 300), device=dev)
    outs = []
    for use_graph in (False, True):
        m.reset()
        rows = list(batched_generate_fn(m, prompts, 300 + 12, prompt_chunksize=64, sample_args=dict(temperature=0.0),
                                        include_prompt=False, use_graph=use_graph))
        outs.append(torch.stack([torch.cat([r[b] for r in rows]) for b in range(B)]))
    assert outs[0].shape == (B, 12) and torch.equal(outs[0], outs[1])


def test_multi_token_chunk_after_decode_steps_reselects():
    """A single-token step selects a handful of slots; a longer chunk that follows selects again from
    the unchanged scores and gets what the full selection would have given."""
    B, C = 2, 256
    cfg, m, dev = _setup("h2o-default", B, C)
    prompts = torch.randint(0, cfg.vocab_size, (B, 300), device=dev)
    with torch.inference_mode():
        _prefill(m, prompts, 500)
        tok = torch.randint(0, cfg.vocab_size, (B, 1), device=dev)
        m(tok)
        cache = m.get_kv_caches()[0]
        few = cache._next_positions.clone()
        assert few.shape[-1] == cache.DECODE_SELECT
        full = cache.next_positions(40).clone()
        assert full.shape[-1] == 40 and torch.equal(full[:, :, : few.shape[-1]], few)
        s = cache.scores[:B, :, : C]
        ref = torch.topk(s, k=40, dim=-1, largest=False, sorted=True)[1].to(torch.int32)
        assert torch.equal(torch.sort(full, -1)[0], torch.sort(ref, -1)[0]) or torch.allclose(
            s.gather(2, full.long()), s.gather(2, ref.long()))
        m(torch.randint(0, cfg.vocab_size, (B, 40), device=dev))  # consumes 40 slots
