"""Builders for gradient tests of cache policies (role of ``keys_values/kvcache/test_utils_advanced.py``): a small
LoRA model with non-trivial adapters, one chunked training step through a named cache, and the same step by the
independent whole-sequence oracle (:mod:`keys_values_b200.oracle`), ready to be compared. Tests of a new policy or a
new buffer type need these three calls and two tolerances."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from keys_values_b200.kvcache.base import KVCacheReplayLog
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.kvcache.gradient.main import LongContextGradientModel
from keys_values_b200.models import lora as lora_mod
from keys_values_b200.models.head_model import CrossEntropyOnLogits, HeadModel


def small_lora_model(seed: int = 0, name: str = "tiny-gpt", lora_r: int = 4, device=None, dtype: torch.dtype = torch.float32,
                     **config_kwargs) -> Tuple[Any, torch.nn.Module]:
    """Random base weights and random (non-zero) LoRA ``B`` factors on q, k, v and the output projection, so that every
    adapter tensor has a gradient that depends on the cache contents."""
    torch.manual_seed(seed)
    cfg = lora_mod.Config.from_name(name, lora_r=lora_r, lora_alpha=2 * lora_r, lora_query=True, lora_key=True, lora_value=True,
                                    lora_projection=True, **config_kwargs)
    model = lora_mod.GPT(cfg)
    model.apply(model._init_weights)
    for n, p in model.named_parameters():
        if "lora_B" in n:
            torch.nn.init.normal_(p, std=0.05)
    lora_mod.mark_only_lora_as_trainable(model)
    if device is not None or dtype != torch.float32:
        model = model.to(device=device, dtype=dtype)
    return cfg, model


@dataclass
class GradientCase:
    """One training step through a cache: what the engine computed and what is needed to replay it elsewhere."""

    model: torch.nn.Module
    head: HeadModel
    input_ids: torch.Tensor
    targets: torch.Tensor
    loss: float
    gradients: Dict[str, torch.Tensor]
    replay_logs: List[KVCacheReplayLog]
    cells: List[Any]

    @property
    def evicts(self) -> bool:
        return any(s is not None for s in self.replay_logs[0].slot_positions)


def run_gradient_case(cache_name: str, batch_size: int = 2, seq_length: int = 200, num_targets: int = 64, cache_length: int = 64,
                      chunk_size: int = 16, layers_per_cell: int = 1, seed: int = 0, model: Optional[torch.nn.Module] = None,
                      cache_kwargs: Optional[Dict[str, Any]] = None, **gradient_kwargs) -> GradientCase:
    """Forward and backward of :class:`LongContextGradientModel` over a random sequence through caches ``cache_name``."""
    if model is None:
        _, model = small_lora_model(seed)
    dev = next(model.parameters()).device
    dtype = next(model.parameters()).dtype
    head = CrossEntropyOnLogits(model.config)
    g = torch.Generator().manual_seed(seed + 1)
    vocab = model.config.vocab_size
    ids = torch.randint(0, vocab, (batch_size, seq_length), generator=g).to(dev)
    tg = torch.randint(0, vocab, (batch_size, num_targets), generator=g).to(dev)
    ck = dict(cache_kwargs or {})
    if "h2o" in cache_name:
        ck.setdefault("max_chunk_size", chunk_size)
    model.assign_kv_caches(KVCacheFactory.create(model, cache_name, batch_size, cache_length, dtype=dtype, device=dev, cache_kwargs=ck or None))
    gm = LongContextGradientModel(model, head, layers_per_cell=layers_per_cell, chunk_size=chunk_size, **gradient_kwargs)
    gm.train()
    loss = gm(ids, tg)
    logs, cells = list(gm._replay_logs), list(gm.cells)
    loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    return GradientCase(model, head, ids, tg, float(loss.value), grads, logs, cells)


def oracle_for(case: GradientCase) -> Tuple[float, Dict[str, torch.Tensor]]:
    """Loss and gradients of the same step by the whole-sequence oracle (masks from the case's replay logs)."""
    from keys_values_b200.oracle import oracle_loss_and_gradients

    loss, grads = oracle_loss_and_gradients(case.model, case.head, case.input_ids, case.targets, case.replay_logs, case.cells)
    return float(loss), grads


def assert_matches_oracle(case: GradientCase, atol: float = 2e-5, rtol: float = 4e-5, loss_tol: float = 2e-5) -> None:
    o_loss, oracle = oracle_for(case)
    assert abs(case.loss - o_loss) < loss_tol, f"loss {case.loss} vs oracle {o_loss}"
    assert case.gradients.keys() == oracle.keys() and case.gradients, "different sets of gradients"
    for k, g in case.gradients.items():
        torch.testing.assert_close(g, oracle[k], atol=atol, rtol=rtol, msg=lambda m_, k=k: f"{k}: {m_}")


def cache_kwargs_for_smart_lastrec(tokenizer, end_initial_regex: str = r"\n\n", max_initial_fraction: float = 0.25, pad_id: int = 0,
                                   **more) -> Dict[str, Any]:
    """Arguments for ``smart-lastrec-*`` caches: the tokens up to the first match of ``end_initial_regex`` in the
    decoded prompt (at most ``max_initial_fraction`` of the slots) are never evicted."""
    return dict(tokenizer=tokenizer, end_initial_regex=end_initial_regex, max_initial_fraction=max_initial_fraction, pad_id=pad_id, **more)
