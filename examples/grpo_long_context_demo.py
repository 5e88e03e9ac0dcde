"""GRPO on long prompts through a bounded KV cache: a self-contained demo.

    python examples/grpo_long_context_demo.py [--steps 3] [--device cpu|cuda]

A tiny random-init model learns to prefer low token ids: prompts of 200 tokens go through an H2O cache of
64 slots (chunked prefill), four completions per prompt are sampled, the reward is the share of generated tokens below a bound,
and the clipped GRPO loss is back-propagated through the eviction decisions with the same cell-wise
backward pass as supervised fine-tuning. Counterpart of ``examples/trl_grpo_demo.ipynb`` of the reference
(which needs the ``trl`` package); see ``docs/USER_GUIDE.md``, section 5.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from keys_values_b200.kvcache.factory import KVCacheFactory  # noqa: E402
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel  # noqa: E402
from keys_values_b200.kvcache.test_utils import MockTokenizer  # noqa: E402
from keys_values_b200.models import lora as lora_mod  # noqa: E402
from keys_values_b200.rl.grpo import GRPOLongContextTrainer, GRPOLossHeadModel  # noqa: E402


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--bound", type=int, default=128, help="tokens with an id below this are rewarded")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    torch.manual_seed(0)
    cfg = lora_mod.Config.from_name("tiny-gpt", lora_r=4, lora_alpha=8, lora_query=True, lora_value=True, lora_head=True)
    gpt = lora_mod.GPT(cfg)
    gpt.apply(gpt._init_weights)
    lora_mod.mark_only_lora_as_trainable(gpt)
    gpt = gpt.to(dev)
    gpt.assign_kv_caches(KVCacheFactory.create(gpt, "h2o-default", 8, 64, device=dev, dtype=torch.float32, cache_kwargs=dict(max_chunk_size=16)))
    head = GRPOLossHeadModel(cfg, epsilon=0.2)
    model = LongContextGradientModel(gpt, head, layers_per_cell=1, chunk_size=16)
    opt = torch.optim.AdamW([p for p in gpt.parameters() if p.requires_grad], lr=5e-3)
    tok = MockTokenizer(vocab_size=cfg.vocab_size, eos_id=None)

    def reward(completion, _meta) -> float:
        return sum(t < a.bound for t in completion) / max(len(completion), 1)

    trainer = GRPOLongContextTrainer(model, opt, tok, reward, num_generations=4, max_new_tokens=8, temperature=1.0)
    prompts = torch.randint(0, cfg.vocab_size, (2, 200), device=dev)
    last = 0.0
    for step in range(a.steps):
        stats = trainer.step(prompts)
        last = stats["mean_reward"]
        print(f"step {step}: loss {stats['loss']:+.4f}  mean reward {stats['mean_reward']:.3f}")
    return last


if __name__ == "__main__":
    main()
