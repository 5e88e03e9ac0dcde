"""The chunked engine against the independent whole-sequence oracle (``keys_values_b200.oracle``): losses and
LoRA gradients through evicting caches, with and without quantized storage; the summed attention weights that
drive the evictions; and the frozen numbers of the tiny reference configuration."""
import json
from pathlib import Path

import pytest
import torch

from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.models import lora as lora_mod
from keys_values_b200.models.head_model import CrossEntropyOnLogits
from keys_values_b200.oracle import oracle_loss_and_gradients, quantize_dequantize, visibility_from_replay_log

DATA = Path(__file__).resolve().parent / "data"


def _lora_model(seed=0, name="tiny-gpt", **kw):
    from keys_values_b200.kvcache.test_utils_advanced import small_lora_model

    return small_lora_model(seed, name, **kw)


def _engine_and_oracle(name, B=2, T=200, n_t=64, C=64, chunk=16, lpc=1, seed=0, **cache_kwargs):
    from keys_values_b200.kvcache.test_utils_advanced import oracle_for, run_gradient_case

    case = run_gradient_case(name, B, T, n_t, C, chunk, lpc, seed, cache_kwargs=cache_kwargs)
    o_loss, oracle = oracle_for(case)
    return case.loss, case.gradients, o_loss, oracle, case.replay_logs, len(case.cells)


@pytest.mark.parametrize("name", ["h2o-default", "h2o-vlen-default", "h2o-orig-default", "lastrec-default"])
@pytest.mark.parametrize("lpc", [1, 2])
def test_gradients_through_eviction_match_oracle(name, lpc):
    """fp32, full-precision buffers: tolerances of the reference's gradient tests (atol 2e-5, rtol 4e-5)."""
    loss, engine, o_loss, oracle, logs, n_cells = _engine_and_oracle(name, lpc=lpc)
    assert n_cells > 2
    assert any(s is not None for s in logs[0].slot_positions), "the sequence must be long enough to evict"
    assert abs(loss - o_loss) < 2e-5
    assert engine.keys() == oracle.keys() and len(engine) > 0
    for k in engine:
        torch.testing.assert_close(engine[k], oracle[k], atol=2e-5, rtol=4e-5, msg=lambda m_: f"{k}: {m_}")


@pytest.mark.parametrize("name", ["h2o-torch-quantized8", "h2o-torch-quantized4", "lastrec-torch-quantized8", "qh2o-torch-quantized8",
                                  "qh2o-vlen-torch-quantized4"])
def test_gradients_with_quantized_storage_match_oracle(name):
    """Rows read from an earlier cell have been through dq(q(x)), rows of the same cell are exact; Q-Hitter
    caches (scores mixed with the quantization error) take part with their recorded decisions."""
    loss, engine, o_loss, oracle, logs, n_cells = _engine_and_oracle(name, B=1)
    assert n_cells > 2
    assert abs(loss - o_loss) < 5e-5
    for k in engine:
        torch.testing.assert_close(engine[k], oracle[k], atol=5e-5, rtol=2e-4, msg=lambda m_: f"{k}: {m_}")


def _eviction_decisions(name, **cache_kwargs):
    from keys_values_b200.long_context import LongContextInferenceModel

    _, m = _lora_model()
    head = CrossEntropyOnLogits(m.config)
    g = torch.Generator().manual_seed(3)
    ids, tg = torch.randint(0, 512, (1, 160), generator=g), torch.randint(0, 512, (1, 16), generator=g)
    m.assign_kv_caches(KVCacheFactory.create(m, name, 1, 48, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=16, **cache_kwargs)))
    for c in m.get_kv_caches():
        c.switch_replay_logging(True)
    with torch.no_grad():
        loss = LongContextInferenceModel(m, head, chunk_size=16)(ids, tg)
    assert torch.isfinite(loss).all()
    caches = m.get_kv_caches()
    return [[s.clone() for s in c.get_replay_log().slot_positions if s is not None] for c in caches], caches


def test_qhitter_follows_its_score_rule():
    """Q-Hitter = H2O scores mixed with the quantization error of each slot,
    ``c·mm(h2o) + ((c − 1)/2)·mm(q_err) + (1 − c)``: with c = 1 the ranking is that of H2O (same evictions on the
    same inputs), with a small c the quantization error takes over and the decisions change."""
    plain, _ = _eviction_decisions("h2o-torch-quantized4")
    same, caches = _eviction_decisions("qh2o-torch-quantized4", combination_constant=1.0)
    mixed, caches_mixed = _eviction_decisions("qh2o-torch-quantized4", combination_constant=0.05)
    assert all(torch.equal(a, b) for la, lb in zip(plain, same) for a, b in zip(la, lb))
    assert any(not torch.equal(a, b) for la, lb in zip(plain, mixed) for a, b in zip(la, lb))
    q_err = caches_mixed[0]._scores["q_errors"]
    assert q_err.shape[-1] == 48 and torch.isfinite(q_err).all() and (q_err > 0).any()


def test_visibility_mask_of_a_hand_made_log():
    from keys_values_b200.kvcache.base import KVCacheReplayLog

    log = KVCacheReplayLog(cache_length=4)
    log.append(4, None)                                 # tokens 0..3 fill slots 0..3
    log.append(2, torch.tensor([[[1, 3]]]))             # tokens 4, 5 replace tokens 1 and 3
    log.append(1, torch.tensor([[[0]]]))                # token 6 replaces token 0
    vis = visibility_from_replay_log(log, 1, 1)[0, 0]
    assert vis[3].tolist() == [True, True, True, True, False, False, False]
    assert vis[4].tolist() == [True, False, True, False, True, False, False]
    assert vis[5].tolist() == [True, False, True, False, True, True, False]
    assert vis[6].tolist() == [False, False, True, False, True, True, True]


def test_quantize_dequantize_round_trip_error():
    x = torch.randn(4, 7, 64)
    for bits, tol in ((8, 0.02), (4, 0.3)):
        err = (quantize_dequantize(x, bits) - x).abs().max()
        span = (x.amax(-1) - x.amin(-1)).max()
        assert err <= span / (2**bits - 1) * 0.5 + 1e-6 and err < tol * span


def test_frozen_numbers_of_the_tiny_configuration():
    """Tiny GPT (2 layers, 64 wide, 4 / 2 heads of 16, vocabulary 512, SwiGLU 172, RoPE base 10000), seed 0, one
    sequence of 512 tokens through H2O caches of 128 slots in chunks of 64, LoRA r = 4: loss, logits, gradient
    norms, evicted slots and 32 greedy tokens stay what they were when ``tests/data/config1.json`` was written,
    and the loss and gradients agree with the oracle."""
    from keys_values_b200.generate.base import generate

    frozen = json.loads((DATA / "config1.json").read_text())
    cur = compute_config1()
    assert cur["evicted_slots_layer0_first_chunks"] == frozen["evicted_slots_layer0_first_chunks"]
    assert cur["greedy_tokens"] == frozen["greedy_tokens"]
    assert abs(cur["loss"] - frozen["loss"]) < 1e-5 and abs(cur["oracle_loss"] - frozen["loss"]) < 2e-5
    torch.testing.assert_close(torch.tensor(cur["last_logits_first8"]), torch.tensor(frozen["last_logits_first8"]), atol=1e-4, rtol=1e-4)
    for k, v in frozen["lora_grad_norms"].items():
        assert abs(cur["lora_grad_norms"][k] - v) <= 1e-5 + 1e-3 * abs(v), k
    assert cur["max_abs_grad_diff_vs_oracle"] < 3e-5


def compute_config1():
    from keys_values_b200.generate.base import generate
    from keys_values_b200.long_context import LongContextInferenceModel

    torch.manual_seed(0)
    cfg = lora_mod.Config(
        name="config1-tiny", block_size=1024, n_layer=2, n_embd=64, n_head=4, n_query_groups=2, head_size=16, vocab_size=512,
        padded_vocab_size=512, norm_class_name="RMSNorm", rotary_percentage=1.0, rope_base=10000, parallel_residual=False, bias=False,
        mlp_class_name="LLaMAMLP", intermediate_size=172, lora_r=4, lora_alpha=8, lora_query=True, lora_key=True, lora_value=True,
        lora_projection=True,
    )
    m = lora_mod.GPT(cfg)
    m.apply(m._init_weights)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(m)
    head = CrossEntropyOnLogits(cfg)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (1, 512), generator=g)
    tg = ids[:, -127:].clone()  # next-token targets of the last 128 positions but one
    tg = torch.cat((tg, torch.randint(0, 512, (1, 1), generator=g)), dim=1)
    m.assign_kv_caches(KVCacheFactory.create(m, "h2o-default", 1, 128, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=64)))
    gm = LongContextGradientModel(m, head, layers_per_cell=1, chunk_size=64)
    gm.train()
    loss = gm(ids, tg)
    logs, cells = list(gm._replay_logs), list(gm.cells)
    evicted = [s[0].tolist() for s in logs[0].slot_positions[1:3]]
    loss.backward()
    grads = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    m.zero_grad()
    o_loss, o_grads = oracle_loss_and_gradients(m, head, ids, tg, logs, cells)
    diff = max(float((grads[k] - o_grads[k]).abs().max()) for k in grads)
    gm.eval()
    with torch.no_grad():
        logits = LongContextInferenceModel(m, head, chunk_size=64)(ids)
        out = generate(m, ids[0], max_returned_tokens=512 + 32, prompt_chunksize=64, temperature=0.0)
    return {
        "loss": float(loss.value), "oracle_loss": float(o_loss), "last_logits_first8": [float(x) for x in logits[0, -1, :8]],
        "lora_grad_norms": {k: float(v.norm()) for k, v in sorted(grads.items())},
        "evicted_slots_layer0_first_chunks": evicted, "greedy_tokens": [int(t) for t in out[-32:]],
        "max_abs_grad_diff_vs_oracle": diff,
    }


if __name__ == "__main__":  # python tests/test_oracle_cpu.py  rewrites the frozen file
    DATA.mkdir(exist_ok=True)
    (DATA / "config1.json").write_text(json.dumps(compute_config1(), indent=1))
    print("written", DATA / "config1.json")


def test_package_builders_for_gradient_tests():
    """The helpers a test of a new policy would use: one call runs the step, one call checks it against the oracle."""
    from keys_values_b200.kvcache.test_utils_advanced import assert_matches_oracle, run_gradient_case

    case = run_gradient_case("h2o-default", batch_size=1, seq_length=160, num_targets=32, cache_length=48, chunk_size=16, layers_per_cell=2)
    assert case.evicts and len(case.cells) > 1 and case.gradients
    assert_matches_oracle(case)
    case.gradients[next(iter(case.gradients))].add_(1e-2)
    with pytest.raises(AssertionError):
        assert_matches_oracle(case)
