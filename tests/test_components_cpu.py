"""Smaller components: checkpoint stores, array-limit ladder, position encodings, replay logs,
adapters (CPU)."""
import math

import pytest
import torch

from keys_values_b200.array_limit import REDUCTION_FACTORS, TemporaryArrayLimit
from keys_values_b200.config import Config
from keys_values_b200.kvcache.base import KVCacheReplayLog
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.checkpoints import KVCheckpoints, LayerInputCheckpoints
from keys_values_b200.models import adapter, adapter_v2
from keys_values_b200.models.model import GPT
from keys_values_b200.models.pos_encoding import (
    LinearPositionEncoding, YaRNPositionEncoding, apply_rope, build_rope_cache, position_encoding_factory,
)


@pytest.mark.parametrize("qname,tol", [(None, 0.0), ("torch-quantized8", 0.02), ("torch-quantized4", 0.3)])
def test_layer_input_checkpoints_round_trip(qname, tol):
    torch.manual_seed(0)
    ck = LayerInputCheckpoints([0, 2], batch_size=2, seq_length=96, n_embd=64, dtype=torch.float32, device="cpu", qname=qname)
    x0, x1 = torch.randn(2, 40, 64), torch.randn(2, 56, 64)
    ck.write(0, 0, 40, x0)
    ck.write(0, 40, 96, x1)
    ck.write(2, 0, 40, -x0)
    for got, want in ((ck.read(0, 0, 40), x0), (ck.read(0, 40, 96), x1), (ck.read(2, 0, 40), -x0)):
        assert got.shape == want.shape
        assert (got - want).abs().max() <= tol * want.abs().max() + 1e-7
    full = 2 * 96 * 64 * 4
    assert ck.size_bytes() > 0 and (qname is None or ck.size_bytes() < full)


def test_kv_checkpoints_keep_snapshots_apart():
    store = KVCheckpoints(offload=False)
    a = {"k": torch.randn(1, 2, 8, 4), "v": torch.randn(1, 2, 8, 4), "token_pos": torch.arange(8).view(1, 1, 8).expand(1, 2, 8), "input_pos": 8}
    b = {"k": torch.randn(1, 2, 8, 4), "v": torch.randn(1, 2, 8, 4), "token_pos": torch.arange(8).view(1, 1, 8).expand(1, 2, 8) + 8, "input_pos": 16}
    store.put(0, 1, a)
    store.put(1, 1, b)
    assert torch.equal(store.get(0, 1)["k"], a["k"]) and store.get(0, 1)["input_pos"] == 8
    assert torch.equal(store.get(1, 1)["token_pos"], b["token_pos"]) and store.get(1, 1)["input_pos"] == 16


def test_array_limit_ladder():
    lim = TemporaryArrayLimit(8.0)
    assert lim() == 8.0
    seen = []
    while lim.can_reduce():
        seen.append(lim.reduce())
    assert seen == [8.0 * f for f in REDUCTION_FACTORS] and lim.reduce() is None
    assert all(a > b for a, b in zip(seen, seen[1:]))
    lim.reset()
    assert lim() == 8.0
    with pytest.raises(ValueError):
        TemporaryArrayLimit(0.0)


def test_rope_tables_and_rotation_are_consistent():
    cos, sin = build_rope_cache(seq_len=32, n_elem=16, base=10000)
    assert cos.shape == (32, 16) and sin.shape == (32, 16)
    torch.testing.assert_close(cos**2 + sin**2, torch.ones_like(cos))
    x = torch.randn(1, 2, 32, 16)
    y = apply_rope(x, cos, sin)
    # a rotation keeps the norm of every (i, i + half) pair, hence of the vector
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5, rtol=1e-5)
    # relative property: <R_m q, R_n k> depends on m - n only
    q, k = torch.randn(16), torch.randn(16)
    def dot(m, n):
        return float((apply_rope(q.view(1, 1, 1, 16), cos[m : m + 1], sin[m : m + 1]) * apply_rope(k.view(1, 1, 1, 16), cos[n : n + 1], sin[n : n + 1])).sum())
    assert abs(dot(5, 3) - dot(12, 10)) < 1e-4 and abs(dot(5, 3) - dot(7, 3)) > 1e-6


def test_yarn_follows_the_context_width():
    cfg = Config.from_name("tiny-gpt")
    lin = LinearPositionEncoding(cfg)
    assert abs(lin.sdpa_scale_factor() - 1 / math.sqrt(cfg.head_size)) < 1e-9
    yarn = position_encoding_factory(cfg, do_yarn=True)
    assert isinstance(yarn, YaRNPositionEncoding)
    yarn.set_context_width(cfg.block_size)
    s1 = yarn.sdpa_scale_factor()
    c1, _ = yarn.tables(0, 8, 0, torch.device("cpu"))
    yarn.set_context_width(8 * cfg.block_size)
    s8 = yarn.sdpa_scale_factor()
    c8, _ = yarn.tables(0, 8, 0, torch.device("cpu"))
    # within the training width YaRN is plain RoPE; beyond it the temperature grows with log(factor)
    # and the low frequencies are interpolated (their angles shrink)
    assert abs(s1 - 1 / math.sqrt(cfg.head_size)) < 1e-6
    want = (0.1 * math.log(8.0) + 1.0) ** 2 / math.sqrt(cfg.head_size)
    assert abs(s8 - want) < 1e-6
    lc, _ = lin.tables(0, 8, 0, torch.device("cpu"))
    torch.testing.assert_close(c1, lc)
    assert not torch.allclose(c8, lc)


def test_replay_log_returns_the_slots_of_a_chunk():
    log = KVCacheReplayLog(cache_length=16)
    log.append(16, None)
    s1 = torch.arange(4, dtype=torch.int32).view(1, 1, 4)
    s2 = (torch.arange(4, dtype=torch.int32) + 7).view(1, 1, 4)
    log.append(4, s1)
    log.append(4, s2)
    assert len(log) == 24 and log.chunk_starts() == [0, 16, 20]
    assert log.slots_for(0, 16) is None
    assert torch.equal(log.slots_for(16, 4), s1) and torch.equal(log.slots_for(20, 4), s2)
    with pytest.raises(Exception):
        log.slots_for(20, 3)


def test_h2o_cache_logs_what_the_replay_needs():
    torch.manual_seed(0)
    cfg = Config.from_name("tiny-gpt")
    m = GPT(cfg)
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 1, 32, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=8)))
    caches = m.get_kv_caches()
    for c in caches:
        c.switch_replay_logging(True)
    ids = torch.randint(0, cfg.vocab_size, (1, 56))
    from keys_values_b200.long_context import LongContextInferenceModel
    from keys_values_b200.models.head_model import CrossEntropyOnLogits

    LongContextInferenceModel(m, CrossEntropyOnLogits(cfg), chunk_size=8)(ids, ids[:, -8:])
    log = caches[0].get_replay_log()
    assert log.token_chunks == [32, 8, 8, 8] and log.slot_positions[0] is None
    for slots in log.slot_positions[1:]:
        assert slots.shape == (1, cfg.n_query_groups, 8)
        # distinct slots inside the cache for every (batch, group)
        assert int(slots.min()) >= 0 and int(slots.max()) < 32
        assert all(len(set(row.tolist())) == 8 for row in slots[0])


def test_adapters_train_only_their_own_parameters():
    torch.manual_seed(0)
    cfg = adapter.Config.from_name("tiny-gpt", adapter_prompt_length=4, adapter_start_layer=0)
    m = adapter.GPT(cfg)
    adapter.mark_only_adapter_as_trainable(m)
    names = [n for n, p in m.named_parameters() if p.requires_grad]
    assert names and all(adapter.adapter_filter(n, None) for n in names)
    ids = torch.randint(0, cfg.vocab_size, (2, 12))
    out = m(ids)
    assert out.shape == (2, 12, cfg.padded_vocab_size) and torch.isfinite(out).all()
    cfg2 = adapter_v2.Config.from_name("tiny-gpt")
    m2 = adapter_v2.GPT(cfg2)
    assert any(isinstance(mod, adapter_v2.AdapterV2Linear) for mod in m2.modules())
    assert m2(ids).shape == (2, 12, cfg2.padded_vocab_size)


def test_adapter_v1_prefix_attention_matches_a_plain_restatement():
    """Gated prefix attention as LitGPT defines it: queries after QK norm and RoPE, prefix keys / values from
    ``qkv(prefix)`` without position encoding, per-head gate, added before the single output projection."""
    import math

    torch.manual_seed(0)
    cfg = adapter.Config.from_name("tiny-qwen3", adapter_prompt_length=5, adapter_start_layer=1, bias=True)
    m = adapter.GPT(cfg)
    m.apply(m._init_weights)
    with torch.no_grad():
        for blk in m.transformer.h:
            torch.nn.init.normal_(blk.attn.proj.bias, std=0.1)
            if hasattr(blk.attn, "gating_factor"):
                torch.nn.init.normal_(blk.attn.gating_factor, std=0.5)
    ids = torch.randint(0, cfg.vocab_size, (2, 24))
    H, G, D = cfg.n_head, cfg.n_query_groups, cfg.head_size

    def plain_attention(attn, x):
        B, T, _ = x.shape
        q, k, v = attn._split_norm_rope(attn.qkv(x), m.mha, 0)  # (B, H|G, T, D), after norm and RoPE
        kr, vr = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
        causal = torch.ones(T, T, dtype=torch.bool).tril()
        att = (q @ kr.transpose(-1, -2)) / math.sqrt(D)
        y = att.masked_fill(~causal, float("-inf")).softmax(-1) @ vr  # (B, H, T, D)
        if attn.block_idx >= cfg.adapter_start_layer:
            _, ak, av = attn.qkv(attn.adapter_wte.weight.unsqueeze(0)).split((H * D, G * D, G * D), dim=-1)
            ak = ak.view(1, -1, G, D).transpose(1, 2).repeat_interleave(H // G, dim=1)  # (1, H, P, D)
            av = av.view(1, -1, G, D).transpose(1, 2).repeat_interleave(H // G, dim=1)
            ay = ((q @ ak.transpose(-1, -2)) / math.sqrt(D)).softmax(-1) @ av
            y = y + attn.gating_factor.view(1, H, 1, 1) * ay
        return attn.proj(y.transpose(1, 2).reshape(B, T, H * D))

    with torch.no_grad():
        x = m.embed(ids)
        for blk in m.transformer.h:
            got = blk.attn(blk.norm_1(x), ids, m.mha)
            want = plain_attention(blk.attn, blk.norm_1(x))
            torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
            x = blk(x, ids, m.mha)


def test_tensor_parallel_sharding_rules_round_trip():
    """Plain and LoRA state dicts: shard over 2 and 4 ranks, put back together, and get the same tensors; the
    shards have the shapes of a model built from the local configuration."""
    from keys_values_b200.config import Config
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.models.model import GPT
    from keys_values_b200.parallel.tp import local_config, shard_state_dict, unshard_state_dict

    torch.manual_seed(0)
    plain_cfg = Config.from_name("tiny-qwen3", n_query_groups=4, bias=True)
    lora_cfg = lora_mod.Config.from_name("tiny-qwen3", n_query_groups=4, lora_r=4, lora_query=True, lora_value=True, lora_projection=True, lora_mlp=True)
    for cfg, cls in ((plain_cfg, GPT), (lora_cfg, lora_mod.GPT)):
        whole = cls(cfg)
        for p in whole.parameters():
            torch.nn.init.normal_(p)
        sd = whole.state_dict()
        for world in (2, 4):
            shards = [shard_state_dict(sd, cfg, world, r) for r in range(world)]
            local = cls(local_config(cfg, world)).state_dict()
            assert all(tuple(shards[0][k].shape) == tuple(local[k].shape) for k in local), "shard shapes"
            back = unshard_state_dict([{k: (v if not k.endswith("proj.bias") or r == 0 else v) for k, v in sh.items()}
                                       for r, sh in enumerate(shards)], cfg)
            assert all(torch.equal(back[k], sd[k]) for k in sd)
            # row-parallel biases live on rank 0 only
            bias_keys = [k for k in sd if k.endswith("attn.proj.bias") or k.endswith("mlp.proj.bias")]
            assert all(float(shards[1][k].abs().sum()) == 0.0 for k in bias_keys)
    with pytest.raises(ValueError):
        local_config(plain_cfg, 3)
