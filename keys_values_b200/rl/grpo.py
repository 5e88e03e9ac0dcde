"""GRPO on long sequences (``keys_values/rl/grpo/{loop,loss,rollout,trainer}.py``).

The clipped policy-gradient loss is a :class:`HeadModel`, so that it goes through the same
chunked forward / cell-wise backward as supervised fine-tuning:
``L = −mean_t min(r_t·A, clip(r_t, 1−ε, 1+ε)·A) + β·KL_t`` with ``r_t = exp(logp_t − logp_old_t)``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from keys_values_b200.config import Config
from keys_values_b200.generate.base import batched_generate_fn
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.models.head_model import IGNORE_INDEX, HeadModel
from keys_values_b200.rl.logprobs import compute_logprobs


def compute_group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-4, scale_rewards: bool = True) -> torch.Tensor:
    """``rewards (num_prompts·group_size,)`` → advantages normalised within each group."""
    r = rewards.view(-1, group_size).float()
    adv = r - r.mean(dim=1, keepdim=True)
    if scale_rewards:
        adv = adv / (r.std(dim=1, keepdim=True) + eps)
    return adv.view(-1)


class GRPOLossHeadModel(HeadModel):
    NAME = "grpo_loss"

    def __init__(self, config: Config, epsilon: float = 0.2, beta: float = 0.0, temperature: float = 1.0):
        super().__init__()
        self._vocab_size = config.padded_vocab_size
        self.epsilon, self.beta, self.temperature = epsilon, beta, temperature
        self.old_logprobs: Optional[torch.Tensor] = None  # (B, num_targets)
        self.ref_logprobs: Optional[torch.Tensor] = None
        self.advantages: Optional[torch.Tensor] = None  # (B,)
        self._num_targets = 0
        self.stats: Dict[str, float] = {}  # sums over the chunks of the last forward pass (see :meth:`pop_stats`)

    def set_batch(self, old_logprobs: torch.Tensor, advantages: torch.Tensor, ref_logprobs: Optional[torch.Tensor] = None) -> None:
        self.old_logprobs, self.advantages, self.ref_logprobs = old_logprobs, advantages, ref_logprobs
        self._num_targets = old_logprobs.shape[1]

    def needs_logits(self) -> bool:
        return True

    def forward(self, model_outputs, targets, input_pos):
        if targets is None:
            return torch.zeros(model_outputs.shape[0], device=model_outputs.device, dtype=torch.float32)
        diff = self._target_offset(model_outputs, targets, self._vocab_size)
        n = targets.shape[1]
        # position of this chunk's targets inside the full target sequence (targets are right-aligned)
        end_pos = input_pos + model_outputs.shape[1]
        total_len = self._total_len
        t_end = self._num_targets - (total_len - end_pos)
        sl = slice(t_end - n, t_end)
        logits = model_outputs[:, diff:, :].float() / self.temperature
        lp = torch.gather(F.log_softmax(logits, dim=-1), 2, targets.clamp(min=0).unsqueeze(-1)).squeeze(-1)
        mask = (targets != IGNORE_INDEX).float()
        ratio = torch.exp(lp - self.old_logprobs[:, sl])
        adv = self.advantages.view(-1, 1)
        loss = -torch.minimum(ratio * adv, ratio.clamp(1 - self.epsilon, 1 + self.epsilon) * adv)
        with torch.no_grad():
            clipped = ((ratio < 1 - self.epsilon) & (adv < 0)) | ((ratio > 1 + self.epsilon) & (adv > 0))
            self._add_stat("clipped", float((clipped.float() * mask).sum()))
            self._add_stat("tokens", float(mask.sum()))
        if self.beta > 0 and self.ref_logprobs is not None:
            d = self.ref_logprobs[:, sl] - lp
            kl = torch.exp(d) - d - 1
            loss = loss + self.beta * kl
            self._add_stat("kl", float((kl.detach() * mask).sum()))
        return (loss * mask).sum(dim=-1)

    def _add_stat(self, name: str, value: float) -> None:
        self.stats[name] = self.stats.get(name, 0.0) + value

    def pop_stats(self) -> Dict[str, float]:
        """Clip fraction and mean KL over the target tokens seen since the last call."""
        n = max(self.stats.get("tokens", 0.0), 1.0)
        out = {"clip_fraction": self.stats.get("clipped", 0.0) / n, "kl": self.stats.get("kl", 0.0) / n}
        self.stats = {}
        return out

    def num_target_entries(self, targets):
        return (targets != IGNORE_INDEX).sum(dim=-1)


@torch.no_grad()
def generate_completions(gpt_model, tokenizer, prompts: torch.Tensor, num_generations: int, max_new_tokens: int, chunk_size: int,
                         temperature: float = 1.0, top_p: float = 1.0) -> List[List[int]]:
    """``num_generations`` sampled completions for every prompt row (rows repeated)."""
    rep = prompts.repeat_interleave(num_generations, dim=0)
    rows: List[List[int]] = [[] for _ in range(rep.shape[0])]
    stop = ([tokenizer.eos_id],) if getattr(tokenizer, "eos_id", None) is not None else ()
    for toks in batched_generate_fn(gpt_model, rep, rep.shape[1] + max_new_tokens, chunk_size, dict(temperature=temperature, top_p=top_p), stop,
                                    include_prompt=False):
        for b, t in enumerate(toks):
            if t is not None:
                rows[b].append(int(t))
    return rows


class adapters_disabled:
    """Context manager: the LoRA branches of ``gpt_model`` are switched off, which turns a LoRA policy into its own
    reference policy (the frozen base model) without a second copy of the weights."""

    def __init__(self, gpt_model):
        from keys_values_b200.models.lora import LoRALinear

        self.layers = [m for m in gpt_model.modules() if isinstance(m, LoRALinear) and m.r > 0]
        self.saved: List[bool] = []

    def __enter__(self):
        self.saved = [m.merged for m in self.layers]
        for m in self.layers:
            if m.merged:
                raise RuntimeError("adapters are merged into the base weights: there is no reference policy to fall back to")
            m.merged = True  # forward() then returns the pretrained branch only
        return self

    def __exit__(self, *exc):
        for m, was in zip(self.layers, self.saved):
            m.merged = was


def grpo_step(model: LongContextGradientModel, optimizer, input_ids: torch.Tensor, targets: torch.Tensor, rewards: torch.Tensor, group_size: int,
              ref_model=None, max_norm: Optional[float] = None, num_iterations: int = 1, scale_rewards: bool = True) -> Dict[str, float]:
    """GRPO update(s) on a batch of (prompt + completion) sequences; ``targets`` hold the completion tokens
    (``-100`` on padding), ``rewards (B,)`` one scalar per sequence. ``num_iterations`` optimisation steps reuse the
    same rollout (the ratio to the sampling policy is what the clipping bounds). With ``beta > 0`` the KL term is
    taken against ``ref_model`` or, if that is ``None`` and the policy has LoRA adapters, against the policy with its
    adapters switched off."""
    head = model.head_model
    if not isinstance(head, GRPOLossHeadModel):
        raise TypeError("model.head_model must be a GRPOLossHeadModel")
    gpt = model.gpt_model
    old = compute_logprobs(gpt, input_ids, targets, model.chunk_size, head.temperature)
    ref = None
    if head.beta > 0:
        if ref_model is not None:
            ref = compute_logprobs(ref_model, input_ids, targets, model.chunk_size, head.temperature)
        else:
            off = adapters_disabled(gpt)
            if off.layers:
                with off:
                    ref = compute_logprobs(gpt, input_ids, targets, model.chunk_size, head.temperature)
    adv = compute_group_advantages(rewards, group_size, scale_rewards=scale_rewards).to(old.device)
    head.set_batch(old, adv, ref)
    head._total_len = input_ids.shape[1]
    head.pop_stats()
    model.train()
    loss = None
    for _ in range(max(1, num_iterations)):
        optimizer.zero_grad(set_to_none=True)
        loss = model(input_ids, targets)
        loss.backward()
        if max_norm is not None:
            torch.nn.utils.clip_grad_norm_([p for g in optimizer.param_groups for p in g["params"] if p.grad is not None], max_norm)
        optimizer.step()
    stats = head.pop_stats()
    lengths = (targets != IGNORE_INDEX).sum(dim=1).float()
    return {"loss": float(loss.detach()), "mean_reward": float(rewards.float().mean()), "reward_std": float(rewards.float().std()) if rewards.numel() > 1 else 0.0,
            "mean_advantage": float(adv.mean()), "mean_completion_length": float(lengths.mean()), **stats}


class GRPOLongContextTrainer:
    """Trainer loop: rollout → rewards → :func:`grpo_step`, with a history of the step statistics. The TRL
    integration of the reference (``rl/grpo/trainer.py``) needs the ``trl`` package, which is optional and absent
    here; this class covers the same loop without it.

    ``reward_fn``: one callable ``(completion_token_ids, meta) -> float`` or a list of them (summed with
    ``reward_weights``); ``num_iterations``: optimisation steps per rollout; ``mask_truncated``: completions that hit
    ``max_new_tokens`` without an end-of-sequence token do not contribute to the loss."""

    def __init__(self, model: LongContextGradientModel, optimizer, tokenizer, reward_fn, num_generations: int = 4, max_new_tokens: int = 64,
                 temperature: float = 1.0, top_p: float = 1.0, reward_weights: Optional[Sequence[float]] = None, num_iterations: int = 1,
                 max_norm: Optional[float] = None, ref_model=None, mask_truncated: bool = False, scale_rewards: bool = True):
        self.model, self.optimizer, self.tokenizer = model, optimizer, tokenizer
        self.reward_fns = list(reward_fn) if isinstance(reward_fn, (list, tuple)) else [reward_fn]
        self.reward_weights = list(reward_weights) if reward_weights is not None else [1.0] * len(self.reward_fns)
        if len(self.reward_weights) != len(self.reward_fns):
            raise ValueError("reward_weights must have one entry per reward function")
        self.num_generations, self.max_new_tokens, self.temperature, self.top_p = num_generations, max_new_tokens, temperature, top_p
        self.num_iterations, self.max_norm, self.ref_model = num_iterations, max_norm, ref_model
        self.mask_truncated, self.scale_rewards = mask_truncated, scale_rewards
        self.history: List[Dict[str, float]] = []

    def rewards(self, completions: List[List[int]], meta: Optional[Sequence[Any]] = None) -> torch.Tensor:
        out = []
        for i, c in enumerate(completions):
            m = None if meta is None else meta[i // self.num_generations]
            out.append(sum(w * float(fn(c, m)) for fn, w in zip(self.reward_fns, self.reward_weights)))
        return torch.tensor(out, dtype=torch.float32)

    def step(self, prompts: torch.Tensor, meta: Optional[Sequence[Any]] = None) -> Dict[str, float]:
        gpt = self.model.gpt_model
        comps = generate_completions(gpt, self.tokenizer, prompts, self.num_generations, self.max_new_tokens, self.model.chunk_size,
                                     self.temperature, self.top_p)
        n = max(max(len(c) for c in comps), 1)
        dev = prompts.device
        rep = prompts.repeat_interleave(self.num_generations, dim=0)
        comp_t = torch.full((len(comps), n), 0, dtype=torch.int64, device=dev)
        tg = torch.full((len(comps), n), IGNORE_INDEX, dtype=torch.int64, device=dev)
        eos = getattr(self.tokenizer, "eos_id", None)
        truncated = 0
        for i, c in enumerate(comps):
            comp_t[i, : len(c)] = torch.tensor(c, device=dev, dtype=torch.int64)
            cut = len(c) >= self.max_new_tokens and (eos is None or not c or c[-1] != eos)
            truncated += int(cut)
            if not (cut and self.mask_truncated):
                tg[i, : len(c)] = torch.tensor(c, device=dev, dtype=torch.int64)
        seq = torch.cat((rep, comp_t), dim=1)
        rewards = self.rewards(comps, meta).to(dev)
        stats = grpo_step(self.model, self.optimizer, seq[:, :-1], tg, rewards, self.num_generations, ref_model=self.ref_model,
                          max_norm=self.max_norm, num_iterations=self.num_iterations, scale_rewards=self.scale_rewards)
        stats["truncated_fraction"] = truncated / max(len(comps), 1)
        self.history.append(stats)
        return stats
