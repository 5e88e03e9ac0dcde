"""Token generation with chunked prefill through bounded KV caches.

The prompt is processed by :class:`LongContextInferenceModel` (prefill chunk of cache
length, then ``chunk_size`` chunks); afterwards tokens are produced one at a time with
``gpt_model(x (B,1))``, which on the GPU runs the single-token decode kernel straight
from the (quantized) cache storage. Parity: ``keys_values/generate/base.py:50-610``.
"""
from __future__ import annotations

from typing import Any, Iterator, List, Optional, Tuple, Union

import torch

from keys_values_b200 import ops as _ops
from keys_values_b200.long_context import LongContextInferenceModel
from keys_values_b200.models.head_model import CrossEntropyOnLogits
from keys_values_b200.models.model import GPT


def multinomial_num_samples_1(probs: torch.Tensor) -> torch.Tensor:
    return torch.multinomial(probs, num_samples=1)


def sample_top_p(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    sorted_logits, sorted_indices = torch.sort(logits, descending=False)
    cumulative = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
    remove = cumulative <= (1 - top_p)
    remove[..., -1:] = False  # keep at least the most likely token
    indices_to_remove = remove.scatter(-1, sorted_indices, remove)
    return logits.masked_fill(indices_to_remove, float("-inf"))


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, top_p: float = 1.0) -> torch.Tensor:
    """Sample one token from ``logits (..., vocab)`` of the last position: top-k filter →
    temperature → top-p filter → multinomial; ``argmax`` when ``temperature == 0``."""
    if top_p < 0.0 or top_p > 1.0:
        raise ValueError(f"top_p must be in [0, 1], got {top_p}")
    logits = logits[0, -1] if logits.ndim == 3 else logits
    if top_k is not None:
        v, i = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = torch.full_like(logits, float("-inf")).scatter_(-1, i, v)
    if temperature > 0.0 and top_k != 1:
        logits = logits / temperature
        if top_p < 1.0:
            logits = sample_top_p(logits, top_p)
        probs = torch.nn.functional.softmax(logits.float(), dim=-1)
        return multinomial_num_samples_1(probs)
    return torch.argmax(logits, dim=-1, keepdim=True)


def next_token(model: GPT, x: torch.Tensor, **sample_kwargs: Any) -> torch.Tensor:
    logits = model(x)
    return sample(logits, **sample_kwargs).to(dtype=torch.int64)


def batched_sample(logits_stack: torch.Tensor, kwargs: Union[dict, List[dict]]) -> torch.Tensor:
    """``logits_stack (B, 1, vocab)``; ``kwargs``: one dict for all rows or one per row."""
    B = logits_stack.shape[0]
    if isinstance(kwargs, dict):
        kwargs = [kwargs] * B
    assert len(kwargs) == B
    if all(kw.get("temperature", 1.0) == 0.0 or kw.get("top_k") == 1 for kw in kwargs):
        from keys_values_b200 import ops

        return ops.argmax_rows(logits_stack[:, -1]).unsqueeze(-1)  # greedy rows: one reduction for the batch
    return torch.stack([sample(logits_stack[b : b + 1], **kw) for b, kw in enumerate(kwargs)], dim=0)


def batched_next_token(model: GPT, x: torch.Tensor, kwargs: Union[dict, List[dict]]) -> torch.Tensor:
    return batched_sample(model(x)[:, -1:], kwargs).to(torch.int64)


def _prefill(model: GPT, prompts: torch.Tensor, chunk_size: int, max_seq_length: int) -> torch.Tensor:
    """Chunked prompt processing; returns the logits of the final prompt position ``(B,1,V)``."""
    lcm = LongContextInferenceModel(model, CrossEntropyOnLogits(model.config), chunk_size=chunk_size)
    lcm.fixed_max_seq_length = max_seq_length
    return lcm(prompts, None)


@torch.inference_mode()
def batched_generate_fn(
    model: GPT,
    prompts: torch.Tensor,
    max_returned_tokens: int,
    prompt_chunksize: int = 1024,
    sample_args: Union[dict, List[dict], None] = None,
    stop_tokens: Tuple[List[int], ...] = (),
    include_prompt: bool = True,
    include_eos: bool = True,
    use_graph: bool = True,
) -> Iterator[List[Optional[torch.Tensor]]]:
    """Yields, step by step, one token (or ``None`` once a row has stopped) per batch row.
    ``prompts (B, T)`` must have equal lengths (left-padded batches). On a GPU the single-token
    steps are replayed from one CUDA graph as soon as all caches are full
    (:class:`keys_values_b200.generate.decode_graph.Decoder`); ``use_graph=False`` keeps them eager."""
    if prompts.ndim == 1:
        prompts = prompts.unsqueeze(0)
    B, T = prompts.shape
    if max_returned_tokens <= T:
        raise ValueError(f"max_returned_tokens = {max_returned_tokens} must exceed the prompt length {T}")
    sample_args = sample_args if sample_args is not None else dict(temperature=0.0)
    if include_prompt:
        for t in range(T):
            yield [prompts[b, t : t + 1] for b in range(B)]
    logits = _prefill(model, prompts, prompt_chunksize, max_returned_tokens)
    tokens = batched_sample(logits, sample_args).view(B, 1).to(torch.int64)
    from keys_values_b200.generate.decode_graph import Decoder

    decoder = Decoder(model, B, use_graph=use_graph and prompts.is_cuda)
    stop_progress = [[0] * len(stop_tokens) for _ in range(B)]
    stopped = [False] * B
    max_stop = max((len(s) for s in stop_tokens), default=0)
    history: List[List[int]] = [[] for _ in range(B)]
    for step in range(max_returned_tokens - T):
        out: List[Optional[torch.Tensor]] = []
        vals = tokens.view(-1).tolist()
        _ops.check_status(tokens.device)  # the host has just waited for the step: a kernel that gave up is reported here
        for b in range(B):
            if stopped[b]:
                out.append(None)
                continue
            history[b].append(vals[b])
            hit = any(len(s) <= len(history[b]) and history[b][-len(s):] == list(s) for s in stop_tokens)
            if hit:
                stopped[b] = True
                out.append(tokens[b] if include_eos else None)
            else:
                out.append(tokens[b])
        yield out
        if all(stopped) or step == max_returned_tokens - T - 1:
            break
        tokens = batched_sample(decoder(tokens)[:, -1:], sample_args).to(torch.int64).view(B, 1)


@torch.inference_mode()
def generate_fn(model: GPT, prompt: torch.Tensor, max_returned_tokens: int, prompt_chunksize: int = 1024, temperature: float = 1.0,
                top_k: Optional[int] = None, top_p: float = 1.0, stop_tokens: Tuple[List[int], ...] = (), include_prompt: bool = True,
                include_eos: bool = True) -> Iterator[torch.Tensor]:
    for toks in batched_generate_fn(model, prompt.view(1, -1), max_returned_tokens, prompt_chunksize,
                                    dict(temperature=temperature, top_k=top_k, top_p=top_p), stop_tokens, include_prompt, include_eos):
        if toks[0] is not None:
            yield toks[0]


@torch.inference_mode()
def generate(model: GPT, prompt: torch.Tensor, max_returned_tokens: int, prompt_chunksize: int = 1024, temperature: float = 1.0,
             top_k: Optional[int] = None, top_p: float = 1.0, eos_id: Optional[int] = None, include_prompt: bool = True) -> torch.Tensor:
    """Generate up to ``max_returned_tokens`` tokens (prompt included) for one prompt."""
    stop = ([eos_id],) if eos_id is not None else ()
    toks = list(generate_fn(model, prompt, max_returned_tokens, prompt_chunksize, temperature, top_k, top_p, stop, include_prompt, True))
    return torch.cat(toks) if toks else torch.empty(0, dtype=torch.int64, device=prompt.device)


def main(checkpoint_dir: str, prompt: str = "What food do llamas eat?", *, max_new_tokens: int = 50, cache_name: str = "h2o-default",
         cache_length: int = 4096, chunk_size: int = 1024, temperature: float = 0.8, top_k: Optional[int] = 50, top_p: float = 1.0,
         precision: Optional[str] = None, device: Optional[str] = None, tp: int = 1, seed: int = 1337) -> Optional[str]:
    """CLI body of ``keys_values_b200 generate``: load a checkpoint directory, generate a reply. ``tp > 1``: the
    model is sharded over ``tp`` ranks of this node (one process per GPU; gloo ranks on a machine without GPUs)."""
    from keys_values_b200.parallel.launch import launch

    result: List[str] = []
    launch(_generate_rank, tp, checkpoint_dir=checkpoint_dir, prompt=prompt, max_new_tokens=max_new_tokens, cache_name=cache_name,
           cache_length=cache_length, chunk_size=chunk_size, temperature=temperature, top_k=top_k, top_p=top_p, precision=precision,
           device=device, seed=seed, result=result)
    return result[0] if result else None  # spawned ranks print the text; it comes back only from an in-process run


def _generate_rank(rank: int, local_rank: int, world: int, *, checkpoint_dir, prompt, max_new_tokens, cache_name, cache_length, chunk_size,
                   temperature, top_k, top_p, precision, device, seed, result) -> None:
    from pathlib import Path

    from keys_values_b200.config import Config
    from keys_values_b200.finetune.utils import load_model_checkpoint
    from keys_values_b200.kvcache.factory import KVCacheFactory
    from keys_values_b200.prompts import has_prompt_style, load_prompt_style, Default
    from keys_values_b200.tokenizer import Tokenizer
    from keys_values_b200.utils import get_default_supported_precision, str_to_torch_dtype

    ckpt = Path(checkpoint_dir)
    if device is not None:
        dev = torch.device(device)
    else:
        dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    dtype = str_to_torch_dtype(precision or get_default_supported_precision(False))
    config = Config.from_checkpoint(ckpt)
    tokenizer = Tokenizer(ckpt)
    style = load_prompt_style(ckpt) if has_prompt_style(ckpt) else Default()
    comm = None
    if world > 1:
        from keys_values_b200.parallel.tp import TPComm, TPGPT, load_sharded_checkpoint

        comm = TPComm(world, rank, dev, dtype=dtype)
        with torch.device(dev):
            model = TPGPT(config, comm)
        model = model.to(dtype)
        load_sharded_checkpoint(model, ckpt)
    else:
        with torch.device(dev):
            model = GPT(config)
        model = model.to(dtype)
        load_model_checkpoint(model, ckpt)
    model.eval()
    torch.manual_seed(seed)  # every rank draws the same samples
    ids = tokenizer.encode(style.apply(prompt), device=dev).to(torch.int64)
    total = ids.numel() + max_new_tokens
    model.max_seq_length = total
    model.assign_kv_caches(KVCacheFactory.create(model, cache_name, 1, min(cache_length, total) if cache_name.startswith("dense") else cache_length,
                                                 device=dev, dtype=dtype))
    out = generate(model, ids, total, chunk_size, temperature, top_k, top_p, eos_id=tokenizer.eos_id, include_prompt=False)
    text = tokenizer.decode(out)
    if rank == 0:
        print(text)
    result.append(text)
    if comm is not None:
        model.close()
        comm.close()
