"""GRPO on long sequences (``keys_values/rl/grpo/{loop,loss,rollout,trainer}.py``).

The clipped policy-gradient loss is a :class:`HeadModel`, so that it goes through the same
chunked forward / cell-wise backward as supervised fine-tuning:
``L = −mean_t min(r_t·A, clip(r_t, 1−ε, 1+ε)·A) + β·KL_t`` with ``r_t = exp(logp_t − logp_old_t)``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence

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
        if self.beta > 0 and self.ref_logprobs is not None:
            d = self.ref_logprobs[:, sl] - lp
            loss = loss + self.beta * (torch.exp(d) - d - 1)
        return (loss * mask).sum(dim=-1)

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


def grpo_step(model: LongContextGradientModel, optimizer, input_ids: torch.Tensor, targets: torch.Tensor, rewards: torch.Tensor, group_size: int,
              ref_model=None, max_norm: Optional[float] = None) -> Dict[str, float]:
    """One GRPO update on a batch of (prompt + completion) sequences; ``targets`` hold the
    completion tokens (``-100`` on padding), ``rewards (B,)`` one scalar per sequence."""
    head = model.head_model
    if not isinstance(head, GRPOLossHeadModel):
        raise TypeError("model.head_model must be a GRPOLossHeadModel")
    gpt = model.gpt_model
    old = compute_logprobs(gpt, input_ids, targets, model.chunk_size, head.temperature)
    ref = compute_logprobs(ref_model, input_ids, targets, model.chunk_size, head.temperature) if ref_model is not None and head.beta > 0 else None
    adv = compute_group_advantages(rewards, group_size).to(old.device)
    head.set_batch(old, adv, ref)
    head._total_len = input_ids.shape[1]
    optimizer.zero_grad(set_to_none=True)
    model.train()
    loss = model(input_ids, targets)
    loss.backward()
    if max_norm is not None:
        torch.nn.utils.clip_grad_norm_([p for g in optimizer.param_groups for p in g["params"] if p.grad is not None], max_norm)
    optimizer.step()
    return {"loss": float(loss.detach()), "mean_reward": float(rewards.float().mean()), "mean_advantage": float(adv.mean())}


class GRPOLongContextTrainer:
    """Minimal trainer loop: rollout → reward → :func:`grpo_step`. The TRL integration of the
    reference (``rl/grpo/trainer.py``) needs the ``trl`` package, which is optional and absent
    here; this class covers the same loop without it."""

    def __init__(self, model: LongContextGradientModel, optimizer, tokenizer, reward_fn: Callable[[List[int], Any], float], num_generations: int = 4,
                 max_new_tokens: int = 64, temperature: float = 1.0):
        self.model, self.optimizer, self.tokenizer, self.reward_fn = model, optimizer, tokenizer, reward_fn
        self.num_generations, self.max_new_tokens, self.temperature = num_generations, max_new_tokens, temperature

    def step(self, prompts: torch.Tensor, meta: Optional[Sequence[Any]] = None) -> Dict[str, float]:
        gpt = self.model.gpt_model
        comps = generate_completions(gpt, self.tokenizer, prompts, self.num_generations, self.max_new_tokens, self.model.chunk_size, self.temperature)
        n = max(len(c) for c in comps)
        dev = prompts.device
        rep = prompts.repeat_interleave(self.num_generations, dim=0)
        comp_t = torch.full((len(comps), n), 0, dtype=torch.int64, device=dev)
        tg = torch.full((len(comps), n), IGNORE_INDEX, dtype=torch.int64, device=dev)
        for i, c in enumerate(comps):
            comp_t[i, : len(c)] = torch.tensor(c, device=dev)
            tg[i, : len(c)] = torch.tensor(c, device=dev)
        seq = torch.cat((rep, comp_t), dim=1)
        rewards = torch.tensor([self.reward_fn(c, None if meta is None else meta[i // self.num_generations]) for i, c in enumerate(comps)], device=dev)
        return grpo_step(self.model, self.optimizer, seq[:, :-1], tg, rewards, self.num_generations)
