"""Small helpers: index utilities, flat-vector access, intermediates recorder, masks, layer stacks, loaders."""
import csv

import pytest
import torch

from keys_values_b200.config import Config
from keys_values_b200.models.model import GPT


def test_misc_utilities(tmp_path):
    from keys_values_b200.utils import misc

    assert misc.find_multiple(512, 128) == 512 and misc.find_multiple(513, 128) == 640
    idx = torch.arange(5)
    i3 = misc.index_to_3d(idx, 2, 3)
    assert i3.shape == (2, 3, 5) and misc.is_index_1d(i3) and not misc.is_index_1d(i3.contiguous())
    assert misc.expand_index(i3, 4).shape == (2, 3, 5, 4)
    x = torch.arange(2 * 2 * 3).view(2, 2, 3)
    assert torch.equal(misc.repeat_interleave(x, 2), x.repeat_interleave(2, dim=1)) and misc.repeat_interleave(x, 1) is x
    torch.manual_seed(0)
    draws = {misc.randint_torch(3, 5) for _ in range(50)}
    assert draws == {3, 4, 5}
    d = {}
    misc.nested_set(d, "a.b.c", 7)
    assert d == {"a": {"b": {"c": 7}}} and misc.nested_get(d, "a.b.c") == 7 and misc.nested_get(d, "a.x", "none") == "none"
    assert misc.str_to_torch_dtype("bf16-true") == torch.bfloat16 and misc.str_to_torch_dtype("32-true") == torch.float32
    with pytest.raises(Exception):
        misc.check_for_nan(torch.tensor([1.0, float("nan")]), "here", "x")
    assert misc.check_for_nan(torch.tensor([1.0]), "here", "x") is False
    path = tmp_path / "rows.csv"
    misc.append_results_to_csv([{"a": 1, "b": 2}], path)
    misc.append_results_to_csv([{"a": 3, "b": 4}], path)
    assert [r["a"] for r in csv.DictReader(open(path))] == ["1", "3"]
    lin = torch.nn.Linear(3, 2)
    lin.bias.requires_grad_(False)
    assert misc.num_parameters(lin) == 8 and misc.num_parameters(lin, True) == 6 and misc.num_parameters(lin, False) == 2
    src, dst = torch.nn.Linear(3, 2), torch.nn.Linear(3, 2)
    misc.copy_parameters(src, dst)
    assert torch.equal(src.weight, dst.weight)


def test_flat_vector_access_round_trip():
    from keys_values_b200.optimize.module_wrapper import AccessWeightsGradients

    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    acc = AccessWeightsGradients(m)
    flat = acc.get_weights()
    assert flat[torch.float32].numel() == sum(p.numel() for p in m.parameters())
    m2 = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    AccessWeightsGradients(m2).set_weights(flat)
    assert all(torch.equal(a, b) for a, b in zip(m.parameters(), m2.parameters()))
    m(torch.randn(5, 4)).sum().backward()
    g = acc.get_gradients()
    acc2 = AccessWeightsGradients(m2)
    acc2.accumulate_gradients(g)
    acc2.accumulate_gradients(g)
    assert all(torch.allclose(2 * a.grad, b.grad) for a, b in zip(m.parameters(), m2.parameters()))
    only = AccessWeightsGradients(m, only_trainable=True)
    m[0].weight.requires_grad_(False)
    assert AccessWeightsGradients(m, only_trainable=True).sizes[torch.float32] == only.sizes[torch.float32] - 12


def test_intermediates_recorder_finds_the_first_difference():
    from keys_values_b200.tools.intermediates import DebugIntermediates

    torch.manual_seed(0)
    cfg = Config.from_name("tiny-gpt")
    a, b = GPT(cfg), GPT(cfg)
    b.load_state_dict(a.state_dict())
    with torch.no_grad():
        b.transformer.h[1].mlp.proj.weight.add_(0.01)
    ids = torch.randint(0, 512, (1, 12))
    ra, rb = DebugIntermediates(lambda n: n.endswith("mlp") or n.endswith("attn")), DebugIntermediates(lambda n: n.endswith("mlp") or n.endswith("attn"))
    ra.register(a)
    rb.register(b)
    with torch.no_grad():
        a(ids), b(ids)
    ra.remove(), rb.remove()
    diff = DebugIntermediates.compare(ra, rb)
    assert diff and diff[0][0].startswith("transformer.h.1.mlp") and all("h.0" not in k for k, _ in diff)
    ra.clear()
    assert not ra.entries


def test_masks_and_sampled_positions():
    from keys_values_b200.attention.attention_utils import build_mask_slice, mask_slice_bool, sample_token_positions, sdpa_attention_weights

    torch.manual_seed(0)
    tp = sample_token_positions(2, 2, 4, 10, 30)
    assert tp.shape == (2, 2, 10) and all(set(range(30, 34)) <= set(tp[b, g].tolist()) for b in range(2) for g in range(2))
    blocked = mask_slice_bool(30, 4, tp, n_head=4)
    assert blocked.shape == (2, 4, 4, 10)
    # query t (position 30 + t) may see every slot whose token is not in its future
    want = tp[:, :, None, :].repeat_interleave(2, dim=1) > (30 + torch.arange(4)).view(1, 1, 4, 1)
    assert torch.equal(blocked, want)
    windowed = mask_slice_bool(30, 4, tp, n_head=4, sliding_window_size=8)
    assert (windowed | ~blocked).all() and windowed.sum() > blocked.sum()
    add = build_mask_slice(30, 4, tp, 4, torch.float32)
    assert (add[blocked] == torch.finfo(torch.float32).min).all() and (add[~blocked] == 0).all()
    q, k, v = torch.randn(2, 4, 4, 16), torch.randn(2, 2, 10, 16), torch.randn(2, 2, 10, 16)
    out, w = sdpa_attention_weights(q, k, v, 0.25, 30, tp)[:2]
    assert out.shape == (2, 4, 4 * 16)[:1] + out.shape[1:] and w.shape == (2, 2, 10)
    assert torch.allclose(w.sum(-1), torch.full((2, 2), 4.0), atol=1e-5)  # every query distributes a weight of one


def test_layer_stack_and_loaders():
    from keys_values_b200.data.dataloader import CycleIterator
    from keys_values_b200.data.trainstate import SeedTrainState
    from keys_values_b200.kvcache.stack_layers import DefaultCellBlocks

    torch.manual_seed(0)
    cfg = Config.from_name("tiny-gpt")
    m = GPT(cfg)
    stack = DefaultCellBlocks(m, first_layer_idx=1, num_layers=1)
    assert stack.first_layer_idx == 1 and stack.num_layers == 1 and stack.blocks() == [m.transformer.h[1]]
    ids = torch.randint(0, 512, (1, 8))
    x = m.embed(ids)
    with torch.no_grad():
        h0 = m.transformer.h[0](x, ids, m.mha)
        assert torch.equal(stack.forward(h0, ids, m.mha), m.transformer.h[1](h0, ids, m.mha))
    it = CycleIterator([1, 2, 3])
    assert [next(it) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1] and it.epoch == 2
    st = SeedTrainState(5)
    other = SeedTrainState(0)
    other.load_state_dict(st.state_dict())
    assert other.seed == 5
