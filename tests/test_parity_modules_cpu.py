"""Modules that mirror smaller parts of the reference: host-resident optimizer, evaluation loaders,
sequence-classification dataset, token-position update, trackers and debug helpers, shard copies."""
import copy

import pytest
import torch

from keys_values_b200.config import Config
from keys_values_b200.models.model import GPT


def _tiny():
    torch.manual_seed(0)
    cfg = Config.from_name("tiny-qwen3")
    m = GPT(cfg)
    m.apply(m._init_weights)
    return cfg, m


def test_host_offload_optimizer_matches_plain_adamw():
    from keys_values_b200.finetune.args import OptimizerArgs

    torch.manual_seed(0)
    net_a = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    net_b = copy.deepcopy(net_a)
    opt_a = OptimizerArgs(learning_rate=1e-2, weight_decay=0.1).create(list(net_a.parameters()))
    opt_b = OptimizerArgs(learning_rate=1e-2, weight_decay=0.1, host_offload=True).create(list(net_b.parameters()))
    assert type(opt_b).__name__ == "HostOffloadOptimizer" and opt_b.param_groups[0]["lr"] == 1e-2
    for step in range(4):
        x = torch.randn(8, 16)
        for net, opt in ((net_a, opt_a), (net_b, opt_b)):
            opt.zero_grad(set_to_none=True)
            net(x).square().mean().backward()
            if step == 2:
                if hasattr(opt, "clip_grad_norm_"):
                    opt.clip_grad_norm_(0.05)
                else:
                    torch.nn.utils.clip_grad_norm_(net.parameters(), 0.05)
            opt.step()
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        torch.testing.assert_close(pa, pb, atol=1e-6, rtol=1e-5)
    # the state round-trips through the checkpoint interface
    st = opt_b.state_dict()
    opt_b.load_state_dict(st)
    assert opt_b.host_bytes() > 0


def test_host_offload_optimizer_keeps_fp32_master_for_bf16_weights():
    from keys_values_b200.optimize.host_optimizer import HostOffloadOptimizer

    w = torch.nn.Parameter(torch.ones(64, dtype=torch.bfloat16))
    opt = HostOffloadOptimizer([w], lambda ps: torch.optim.SGD(ps, lr=1e-3))
    for _ in range(10):  # ten updates of 1e-3 · 0.25: each is below bf16 resolution at 1.0, their sum is not
        opt.zero_grad()
        w.grad = torch.full_like(w, 0.25)
        opt.step()
    assert abs(float(opt.host_params[0].detach()[0]) - (1 - 10 * 2.5e-4)) < 1e-6
    assert float(w.detach()[0]) < 1.0  # the accumulated change reached the bf16 copy


def test_evaluation_loader_orders_tasks_and_lengths():
    from keys_values_b200.data.constants import ORIG_IDX_NAME, TASK_NAME
    from keys_values_b200.data.evaluation import EvaluationDataLoader, SimilarSequenceLengthWithTasksSampler

    lengths = [50, 10, 40, 20, 30]
    sampler = SimilarSequenceLengthWithTasksSampler(lengths, micro_batch_size=2, num_tasks=2)
    assert len(sampler) == 6 and sampler.batch_size == 2
    dataset = [{"x": i} for i in range(5)] + [{"__pad__": True}]
    loader = EvaluationDataLoader(dataset, sampler, lambda items: {"items": items}, ["ckpt_a", "ckpt_b"], delay_tokenization=True)
    jobs = list(loader)
    assert [j[TASK_NAME] for j in jobs] == ["ckpt_a"] * 3 + ["ckpt_b"] * 3
    assert [j[ORIG_IDX_NAME] for j in jobs[:3]] == [[1, 3], [4, 2], [0, 5]]  # shortest first, pad entry last
    assert "items" not in jobs[0]
    full = iter(loader).fetch_full(jobs[1])
    assert [it["x"] for it in full["items"]] == [4, 2]
    with pytest.raises(ValueError):
        list(EvaluationDataLoader(dataset[:5], sampler, lambda x: x, ["a", "b"]))


def test_sequence_classification_dataset_and_collate():
    from keys_values_b200.data.sequence_classification import SequenceClassificationDataset, get_seq_class_collate_fn

    class Tok:
        def encode(self, text, bos=False, eos=False, max_length=-1):
            ids = [ord(ch) % 50 for ch in text] + ([1] if eos else [])
            return torch.tensor(ids[:max_length] if max_length > 0 else ids)

    data = [dict(instruction="abc", output="yes"), dict(instruction="defgh", output="no"), {"__pad__": True}]
    ds = SequenceClassificationDataset(data, Tok(), None, ["no", "yes"])
    assert ds[0]["labels"] == 1 and ds[1]["labels"] == 0 and ds[0]["input_ids"].tolist()[-1] == 1
    assert ds[0]["token_counts"] == {"raw_plus_prompt_template": 4, "raw": 4}
    batch = get_seq_class_collate_fn(pad_id=0)([ds[0], ds[1], ds[2]])
    assert batch["input_ids"].shape == (2, 6) and batch["labels"].tolist() == [1, 0]
    with pytest.raises(ValueError):
        SequenceClassificationDataset([dict(instruction="a", output="maybe")], Tok(), None, ["no", "yes"])
    with pytest.raises(ValueError):
        SequenceClassificationDataset([{"__pad__": True}, dict(instruction="a", output="no")], Tok(), None, ["no", "yes"])


def test_update_token_positions_matches_cache_state():
    from keys_values_b200.kvcache.attn_weights import update_token_positions

    tp = torch.zeros(2, 2, 8, dtype=torch.int32)
    assert update_token_positions(tp, 0, 8, 2, None) is None
    assert tp[1, 1].tolist() == list(range(8))
    index = torch.tensor([[[3, 5], [0, 1]], [[7, 6], [2, 4]]], dtype=torch.int32)
    update_token_positions(tp, 8, 2, 2, index)
    assert tp[0, 0].tolist() == [0, 1, 2, 8, 4, 9, 6, 7] and tp[1, 1].tolist() == [0, 1, 10 - 2, 3, 9, 5, 6, 7]
    # grace ring of 2 slots (6, 7): the oldest ring entry moves to the evicted slot, the new token takes its place
    tp = torch.arange(8, dtype=torch.int32).view(1, 1, 8).repeat(1, 1, 1)
    ring, n1, prefix = update_token_positions(tp, 8, 1, 1, torch.tensor([[[2]]], dtype=torch.int32), grace_period=2, next_grace_pos=6)
    assert (n1, prefix) == (0, 6) and ring.tolist() == [[[6]]]
    assert tp[0, 0].tolist() == [0, 1, 6, 3, 4, 5, 8, 7]


def test_tracker_and_debug_utils(tmp_path):
    from keys_values_b200.tools import debug_utils as du
    from keys_values_b200.tools import tracker

    x = torch.randn(100)
    assert tracker.track(x) is x  # disarmed
    f = tmp_path / "bad.pt"
    tracker.initialize_weights_tracker(str(f), threshold=50.0)
    try:
        assert tracker.track(x, "fine") is x
        y = x.clone()
        y[3] = float("nan")
        tracker.set_message_postfix("layer 3")
        with pytest.raises(AssertionError, match="1 of 100 entries are NaN: here: layer 3"):
            tracker.track(y, "here")
        assert torch.isnan(torch.load(f)[3])
        with pytest.raises(AssertionError, match=r"\|elem\| > 50"):
            tracker.track(x * 1e4)
        lin = torch.nn.Linear(4, 4)
        tracker.set_message_postfix(None)
        tracker.track_weights(lin, "after step")
    finally:
        tracker.initialize_weights_tracker(None)
    v = torch.arange(101, dtype=torch.float32)
    for q in (0.0, 0.01, 0.5, 0.9, 1.0):
        torch.testing.assert_close(du.torch_quantile(v, q), torch.quantile(v, q))
    m = torch.randn(7, 33)
    torch.testing.assert_close(du.torch_quantile(m, 0.3, dim=1), torch.quantile(m, 0.3, dim=1))
    assert du.size_quantiles(v).count("|") == 3 and du.for_debug(v).device.type == "cpu"
    du.debug_compare_dicts({"a": v}, {"a": v.clone()})
    with pytest.raises(AssertionError):
        du.debug_compare_dicts({"a": v}, {"a": v + 1})
    with pytest.raises(ValueError):
        du.debug_compare_dicts({"a": v}, {"b": v})


def test_shard_cell_block_and_replay_logs():
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.kvcache.gradient import get_replay_logs
    from keys_values_b200.optimize.grad_accumulate import DistributedPrimitives
    from keys_values_b200.optimize.model_factory import GPTShardCellBlock

    cfg, m = _tiny()
    shard = GPTShardCellBlock(m, "h0:2", "cpu")
    assert (shard.first_layer_idx, shard.num_layers) == (0, 2)
    x = torch.randn(1, 6, cfg.n_embd, requires_grad=True)
    idx = torch.randint(0, cfg.vocab_size, (1, 6))
    y = shard(x, idx, m.mha)
    y_ref = x
    for b in m.transformer.h:
        y_ref = b(y_ref, idx, m.mha)
    torch.testing.assert_close(y, y_ref)
    y.sum().backward()
    shard.return_gradients()
    assert all(p.grad is not None for p in m.transformer.h[1].parameters())
    with pytest.raises(ValueError):
        GPTShardCellBlock(m, "wte", "cpu")
    caches = KVCacheFactory.create(m, "h2o-default", 1, 16, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=4))
    m.assign_kv_caches(caches)
    with pytest.raises(IndexError):
        get_replay_logs(m)
    for c in caches:
        c.switch_replay_logging(True)
    m.max_seq_length = 64
    with torch.no_grad():
        m(torch.randint(0, cfg.vocab_size, (1, 16)))
        m(torch.randint(0, cfg.vocab_size, (1, 4)))
    logs = get_replay_logs(m)
    assert len(logs) == cfg.n_layer and all(log is not None for log in logs)
    assert DistributedPrimitives.world_size() == 1 and DistributedPrimitives.rank() == 0
    t = torch.ones(3)
    DistributedPrimitives.all_reduce_mean(t)
    assert t.tolist() == [1, 1, 1]


def test_sample_metric_on_loader_generates_and_scores():
    from keys_values_b200.evaluation.evaluator import sample_metric_on_loader, split_prompts_and_references
    from keys_values_b200.kvcache.factory import KVCacheFactory

    class Tok:
        eos_id, pad_id = 1, 0

        def decode(self, ids):
            return " ".join(str(int(i)) for i in ids)

    cfg, m = _tiny()
    m.eval()
    ids = torch.tensor([[5, 6, 7, 8, 9, 1, 0, 0], [11, 12, 13, 14, 15, 16, 17, 1]])
    labels = torch.full_like(ids, -100)
    labels[0, 4:6] = ids[0, 4:6]
    labels[1, 6:8] = ids[1, 6:8]
    batch = {"input_ids": ids, "labels": labels}
    prompts, refs = split_prompts_and_references(batch, Tok())
    assert prompts.tolist() == [[0, 0, 5, 6, 7, 8], [11, 12, 13, 14, 15, 16]] and refs == [["9"], ["17"]]
    m.assign_kv_caches(KVCacheFactory.create(m, "dense-default", 2, 32, dtype=torch.float32))
    seen = []
    res = sample_metric_on_loader(m, Tok(), [batch, batch], "exact_match", torch.device("cpu"), max_batches=1, max_new_tokens=3,
                                  prompt_chunksize=4, on_batch=lambda k, r: seen.append((k, r["generated"], r["references"])))
    assert res["num_samples"] == 2 and 0.0 <= res["mean"] <= 1.0
    assert len(seen) == 1 and len(seen[0][1]) == 2 and seen[0][2] == ["9", "17"]


def test_merge_lora_and_peft_import(tmp_path):
    import yaml

    from keys_values_b200.finetune.utils import LIT_MODEL_FNAME, load_model_checkpoint, save_model_checkpoint
    from keys_values_b200.models import lora as lora_mod
    from keys_values_b200.tools import merge_lora

    base_cfg = Config.from_name("tiny-gpt")
    torch.manual_seed(0)
    base = GPT(base_cfg)
    base.apply(base._init_weights)
    base_dir = tmp_path / "base"
    base_dir.mkdir()
    base_cfg.save(base_dir / "model_config.yaml")
    torch.save({"model": base.state_dict()}, base_dir / LIT_MODEL_FNAME)
    largs = dict(r=4, alpha=8, dropout=0.0, query=True, key=False, value=True, projection=True, mlp=False, head=False)
    lcfg = lora_mod.Config.from_checkpoint(base_dir, lora_r=4, lora_alpha=8, lora_query=True, lora_value=True, lora_projection=True)
    lm = lora_mod.GPT(lcfg)
    load_model_checkpoint(lm, base_dir)
    for n, p in lm.named_parameters():
        if "lora_" in n:
            torch.nn.init.normal_(p, std=0.05)
    fin = tmp_path / "out" / "final"
    save_model_checkpoint(lm, None, fin, lora=True)
    (fin / "hyperparameters.yaml").write_text(yaml.safe_dump({"lora": largs}))
    ids = torch.randint(0, base_cfg.vocab_size, (1, 12))
    lm.eval()
    with torch.no_grad():
        want = lm(ids)
    merged_dir = merge_lora.merge(fin, base_dir)
    plain = GPT(Config.from_checkpoint(merged_dir))
    load_model_checkpoint(plain, merged_dir)
    plain.eval()
    with torch.no_grad():
        torch.testing.assert_close(plain(ids), want, atol=1e-5, rtol=1e-4)
    with torch.no_grad():
        assert float((plain(ids) - base.eval()(ids)).abs().max()) > 1e-4  # the adapter did change the model

    # PEFT layout → fused qkv adapters: same tensors, stacked in q, v order
    qkv = lm.transformer.h[0].attn.qkv
    r = 4
    A, B = qkv.lora_A.detach(), qkv.lora_B.detach()
    q_out = base_cfg.n_head * base_cfg.head_size
    peft = {
        "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": A[:r], "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": B[:q_out],
        "base_model.model.model.layers.0.self_attn.v_proj.lora_A.default.weight": A[r:], "base_model.model.model.layers.0.self_attn.v_proj.lora_B.default.weight": B[q_out:],
        "base_model.model.model.layers.0.self_attn.o_proj.lora_A.weight": lm.transformer.h[0].attn.proj.lora_A.detach(),
        "base_model.model.model.layers.0.self_attn.o_proj.lora_B.weight": lm.transformer.h[0].attn.proj.lora_B.detach(),
    }
    sd = merge_lora.peft_to_lora_state_dict(peft, ("q_proj", "v_proj"))
    torch.testing.assert_close(sd["transformer.h.0.attn.qkv.lora_A"], A)
    torch.testing.assert_close(sd["transformer.h.0.attn.qkv.lora_B"], B)
    assert "transformer.h.0.attn.proj.lora_B" in sd
    with pytest.raises(ValueError):
        merge_lora.peft_to_lora_state_dict(peft, ("q_proj", "k_proj", "v_proj"))


def test_experiment_files_and_token_counts(tmp_path):
    import csv

    import yaml

    from keys_values_b200.tools import dataset_token_counts as dtc
    from keys_values_b200.tools import experiment_files as ef

    ev = tmp_path / "run" / "h2o-default__final" / "eval"
    ev.mkdir(parents=True)
    for b, (loss, score) in enumerate(((2.0, 1.0), (4.0, 0.0))):
        with open(ev / f"eval_metrics_{b}.csv", "w", newline="") as fp:
            w = csv.DictWriter(fp, fieldnames=["task", "batch", "row", "loss", "num_tokens", "time", "exact_match"])
            w.writeheader()
            w.writerow(dict(task="h2o-default__final", batch=b, row=0, loss=loss, num_tokens=100 * (b + 1), time=1.5, exact_match=score))
        (ev / f"generated_samples_{b}.yaml").write_text(yaml.safe_dump({"reference": "a b", "generated": "a b c d", "score": score}) + "---\n")
    (ev / "batch_7.lock").write_text("123")
    run = tmp_path / "run"
    table = ef.result_table(run)
    assert len(table) == 1 and abs(table[0]["loss"] - (2 * 100 + 4 * 200) / 300) < 1e-9 and table[0]["exact_match"] == 0.5 and table[0]["time"] == 3.0
    assert (run / ef.METRICS_ALL).is_file()
    assert ef.collect_gen_samples(run) == {"h2o-default__final": 2}
    stats = ef.sample_stats(run)
    assert stats[0]["samples"] == 2 and stats[0]["length_ratio_mean"] == 2.0 and stats[0]["score_mean"] == 0.5
    assert ef.cleanup_evaluation(run) == 1 and not (ev / "batch_7.lock").exists() and (ev / "eval_metrics_0.csv").exists()
    assert ef.cleanup_gen_samples(run) == 2 and (ev / ef.SAMPLES_ALL).exists()
    (run / "metrics.csv").write_text("step,loss,val_loss\n1,3.0,\n2,2.5,2.75\n4,2.0,2.5\n")
    assert ef.collect_val_loss(run) == {2: 2.75, 4: 2.5} and (run / "val_losses.yaml").is_file()
    step = run / "step-000002"
    step.mkdir()
    for name in ("lit_model.lora.pth", "tokenizer.json", "training_state.pt"):
        (step / name).write_text("x")
    assert ef.strip_checkpoints(run) == 2 and (step / "lit_model.lora.pth").exists()
    jl = tmp_path / "evaluation.jsonl"
    jl.write_text('{"answer": "x", "prediction": "y z"}\n')
    assert ef.convert_samples(jl, tmp_path / "s.yaml") == 1 and "y z" in (tmp_path / "s.yaml").read_text()
    ef.main(["result-table", str(run)])
    # token counts
    data = tmp_path / "d.jsonl"
    data.write_text('{"instruction": "a b c", "output": "d"}\n{"instruction": "a", "output": "b"}\n')
    counts = dtc.token_counts(dtc.load_records(data), lambda s: s.split(), ["instruction", "output"])
    assert counts == [4, 2] and dtc.summarize(counts)["max"] == 4


def test_kvcache_test_utils():
    from keys_values_b200.attention.base import DefaultKeysAndValues
    from keys_values_b200.kvcache import test_utils as tu
    from keys_values_b200.kvcache.base import KVCacheParams

    params = KVCacheParams(max_batch_size=2, n_query_groups=2, cache_length=16, head_size=8, n_head=4, dtype=torch.float32)
    cache = tu.create_kv_cache("h2o-default", params, max_chunk_size=4)
    log = tu.record_forward_calls(cache)
    args = tu.random_args_cache_forward(params, 20, vocab_size=50)
    out0 = cache(**tu.range_from_args(args, 0, 16))
    out1 = cache(**tu.range_from_args(args, 16, 20))
    assert out0.shape == (2, 16, 32) and out1.shape == (2, 4, 32)
    assert [c.inputs.input_pos for c in log] == [0, 16] and log[1].token_positions.shape == (2, 2, 16)
    idx = tu.random_index(params, 4, 12, 5)
    assert idx.shape == (2, 2, 5) and int(idx.min()) >= 4 and int(idx.max()) < 12
    assert all(len(set(r.tolist())) == 5 for r in idx.view(-1, 5))
    q, (k, v) = tu.random_tensor(params, 3, is_query=True), tu.random_keys_values(params, 10)
    w = tu.compute_attn_weights(q, DefaultKeysAndValues(k, v))
    assert w.shape == (2, 2, 10) and torch.allclose(w.sum(-1), torch.full((2, 2), 3.0), atol=1e-4)
    m = tu.attention_mask_forward(3, 5, torch.float32)
    assert m.shape == (1, 1, 3, 5) and float(m[0, 0, 0, 3]) < -1e30 and float(m[0, 0, 2, 4]) == 0.0 and tu.attention_mask_forward(1, 5, torch.float32) is None
    assert tu.tensor_is_simple(q) and not tu.tensor_is_simple(q[:, :1].expand(2, 4, 3, 8))
    names = tu.cache_names_and_devices(["h2o-default", "dense-bnb-quantized8"])
    assert ("h2o-default", torch.device("cpu")) in names and all("bnb" not in n or tu.have_bitsandbytes() for n, _ in names)
    tok = tu.MockTokenizer()
    assert tok.encode(tu.sequence_of_words(5), eos=True).tolist()[-1] == tok.eos_id and len(tu.product_with_devices([1, 2], ["a"])) >= 2


def test_profile_caches_tool_on_cpu():
    from keys_values_b200.tools.profile_caches import profile

    rows = profile("tiny-gpt", ["dense-default", "lastrec-default", "h2o-torch-quantized8", "no-such-cache"], batch=1, seq_len=96,
                   cache_length=32, chunk_size=8, device=torch.device("cpu"), dtype=torch.float32)
    assert [r["cache"] for r in rows] == ["dense-default", "lastrec-default", "h2o-torch-quantized8", "no-such-cache"]
    assert all(r["tokens_per_s"] > 0 for r in rows[:3]) and "error" in rows[3]


def test_analyze_gradient_data(tmp_path):
    from keys_values_b200.tools import analyze_gradient_data as agd

    torch.manual_seed(0)
    nets = [torch.nn.Linear(4, 3) for _ in range(2)]
    nets[1].load_state_dict(nets[0].state_dict())
    befores = []
    for r, net in enumerate(nets):
        net(torch.randn(5, 4)).sum().backward()
        befores.append(agd.record_gradients(net, lambda n: n == "weight"))
    mean = {k: (befores[0][k] + befores[1][k]) / 2 for k in befores[0]}
    for r in range(2):
        agd.save_record(tmp_path, 0, r, befores[r], mean)
    recs = agd.load_records(tmp_path, 0, 2)
    agd.check_consistency(recs, "iteration 0")
    agd.main([str(tmp_path), "--iters", "0", "--devices", "2"])
    agd.save_record(tmp_path, 1, 0, befores[0], mean)
    agd.save_record(tmp_path, 1, 1, befores[1], {k: v * 1.5 for k, v in mean.items()})
    with pytest.raises(ValueError, match="differs between rank 0 and rank 1"):
        agd.check_consistency(agd.load_records(tmp_path, 1, 2), "iteration 1")
    assert "zeros: 1 of 4" in agd.text_histogram(torch.tensor([0.0, 1e-3, 1e-2, 1.0]))
