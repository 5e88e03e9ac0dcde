"""Helpers for testing KV caches: random inputs in the shapes a cache expects, single caches without
a model, device enumeration, a mock tokenizer, and a recorder of a cache's calls. They live in the
package (not under ``tests/``) so that code extending the cache policies can use them
(``keys_values/kvcache/test_utils.py:37-319``, ``test_utils_advanced.py:110-180``,
``test_before_after.py:27-140``).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from keys_values_b200.attention.base import KeysAndValues
from keys_values_b200.config import Config
from keys_values_b200.kvcache.base import KVCache, KVCacheParams
from keys_values_b200.kvcache.factory import KVCacheFactory
from keys_values_b200.ops import reference as ref


def create_kv_cache(name: str, params: KVCacheParams, block_idx: int = 0, device=None, **kwargs) -> KVCache:
    """A single cache named ``name`` for the geometry of ``params`` (no model needed)."""
    config = Config(n_embd=params.n_head * params.head_size, n_head=params.n_head, n_query_groups=params.n_query_groups, n_layer=1,
                    head_size=params.head_size)
    return KVCacheFactory.create_single(name=name, config=config, max_batch_size=params.max_batch_size, cache_length=params.cache_length,
                                        block_idx=block_idx, device=device, dtype=params.dtype, cache_kwargs=kwargs)


def tensor_is_simple(x: torch.Tensor) -> bool:
    """Contiguous and not a broadcast view."""
    return x.is_contiguous() and all(st != 0 for st, n in zip(x.stride(), x.shape) if n > 1)


def random_tensor(params: KVCacheParams, num: int, is_query: bool = False, device=None, batch_size: Optional[int] = None) -> torch.Tensor:
    heads = params.n_head if is_query else params.n_query_groups
    B = params.max_batch_size if batch_size is None else batch_size
    return torch.randn((B, heads, num, params.head_size), dtype=params.dtype or torch.float32, device=device)


def random_keys_values(params: KVCacheParams, num: int, device=None, batch_size: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    return random_tensor(params, num, device=device, batch_size=batch_size), random_tensor(params, num, device=device, batch_size=batch_size)


def random_args_cache_forward(params: KVCacheParams, num: int, vocab_size: Optional[int] = None, device=None) -> Dict[str, torch.Tensor]:
    """Keyword arguments of ``KVCache.forward`` for ``num`` new tokens."""
    k, v = random_keys_values(params, num, device)
    out = {"query": random_tensor(params, num, True, device), "key": k, "value": v}
    if vocab_size is not None:
        out["token_idx"] = torch.randint(0, vocab_size, (params.max_batch_size, num), device=device)
    return out


def range_from_args(data: Dict[str, torch.Tensor], start: int, end: int, only_query: bool = False) -> Dict[str, torch.Tensor]:
    """Tokens ``[start, end)`` of forward arguments (with ``only_query`` the keys/values stay whole)."""
    out = {"query": data["query"][:, :, start:end]}
    for name in ("key", "value"):
        out[name] = data[name] if only_query else data[name][:, :, start:end]
    if "token_idx" in data:
        out["token_idx"] = data["token_idx"] if only_query else data["token_idx"][:, start:end]
    return out


def random_index(params: KVCacheParams, start: int, end: int, num: int, batch_size: Optional[int] = None, device=None) -> torch.Tensor:
    """``(B, G, num)`` int32 slots in ``[start, end)``, distinct within each (b, g)."""
    B = params.max_batch_size if batch_size is None else batch_size
    if num > end - start:
        raise ValueError(f"cannot draw {num} distinct slots from [{start}, {end})")
    rows = [torch.randperm(end - start, device=device)[:num] + start for _ in range(B * params.n_query_groups)]
    return torch.stack(rows).view(B, params.n_query_groups, num).to(torch.int32)


def attention_mask_forward(q_len: int, k_len: int, dtype: torch.dtype, device=None) -> Optional[torch.Tensor]:
    """Additive causal mask ``(1,1,q_len,k_len)`` for queries that are the last ``q_len`` of ``k_len`` positions."""
    if q_len > k_len:
        raise ValueError("q_len must not exceed k_len")
    if q_len <= 1:
        return None
    future = torch.ones(q_len, q_len, dtype=torch.bool, device=device).triu(diagonal=1)
    mask = torch.zeros(q_len, k_len, dtype=dtype, device=device)
    mask[:, k_len - q_len :].masked_fill_(future, torch.finfo(dtype).min)
    return mask.view(1, 1, q_len, k_len)


def compute_attn_weights(query: torch.Tensor, k_and_v: KeysAndValues, token_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Summed attention weights ``(B, G, kv_len)`` of causal attention with the queries at the end
    (fp32 restatement: sum over queries, mean over the heads of a group)."""
    k, v = k_and_v.keys(), k_and_v.values()
    q_len, kv_len = query.shape[2], k.shape[2]
    _, w = ref.sdpa(query, k, v, 1.0 / math.sqrt(query.shape[-1]), kv_len - q_len, token_positions, True)[:2]
    return w


def copy_gradients(model: torch.nn.Module, device=None) -> Dict[str, torch.Tensor]:
    return {n: p.grad.detach().clone().to(device or p.grad.device) for n, p in model.named_parameters() if p.grad is not None}


def debug_print_gradients(model: torch.nn.Module) -> None:
    for n, p in model.named_parameters():
        if p.grad is not None:
            print(f"{n}: |grad| max {float(p.grad.abs().max()):.3e}, mean {float(p.grad.abs().mean()):.3e}")


def have_bitsandbytes() -> bool:
    try:
        import bitsandbytes  # noqa: F401

        return torch.cuda.is_available()
    except ImportError:
        return False


def available_backends() -> List[torch.device]:
    devs = [torch.device("cpu")]
    if torch.cuda.is_available():
        devs.append(torch.device("cuda", 0))
    return devs


def cache_name_is_bitsandbytes(name: str) -> bool:
    return "-bnb-" in name


def cache_name_gpu_only(name: str) -> bool:
    return cache_name_is_bitsandbytes(name)


def device_for_cache_name(name: str) -> torch.device:
    return torch.device("cuda", 0) if cache_name_gpu_only(name) else torch.device("cpu")


def filter_cache_names(names: Iterable[str]) -> List[str]:
    """Drops the names whose quantizer is not installed or has no device here."""
    return [n for n in names if not cache_name_is_bitsandbytes(n) or have_bitsandbytes()]


def cache_names_and_devices(names: Optional[Iterable[str]] = None) -> List[Tuple[str, torch.device]]:
    names = filter_cache_names(KVCacheFactory.supported_names() if names is None else names)
    return [(n, d) for n in names for d in available_backends() if not (cache_name_gpu_only(n) and d.type != "cuda")]


def product_with_devices(*lists: Sequence[Any]) -> List[Tuple[Any, ...]]:
    return [(*combo, d) for combo in itertools.product(*lists) for d in available_backends()]


class MockTokenizer:
    """Words are the tokens: enough of a tokenizer for caches that look at the decoded prompt."""

    def __init__(self, vocab_size: int = 1000, eos_id: int = 1, pad_id: int = 0):
        self.vocab_size, self.eos_id, self.pad_id, self.bos_id = vocab_size, eos_id, pad_id, None

    def encode(self, text: str, bos: bool = False, eos: bool = False, max_length: int = -1, device=None) -> torch.Tensor:
        ids = [2 + (sum(map(ord, w)) % (self.vocab_size - 2)) for w in text.split()]
        if eos:
            ids.append(self.eos_id)
        if max_length > 0:
            ids = ids[:max_length]
        return torch.tensor(ids, dtype=torch.int64, device=device)

    def decode(self, ids) -> str:
        return " ".join(f"w{int(i)}" for i in ids)


def sequence_of_words(num_words: int) -> str:
    return " ".join(f"word{i % 97}" for i in range(num_words))


@dataclass
class ForwardInput:
    """Arguments of one ``KVCache.forward`` call (detached CPU copies)."""

    query: torch.Tensor
    key: torch.Tensor
    value: torch.Tensor
    token_idx: Optional[torch.Tensor]
    input_pos: int


@dataclass
class ForwardInputOutput:
    inputs: ForwardInput
    output: torch.Tensor
    token_positions: Optional[torch.Tensor] = None
    extra: Dict[str, Any] = field(default_factory=dict)


def record_forward_calls(cache: KVCache) -> List[ForwardInputOutput]:
    """Wraps ``cache.forward`` so that every call is appended to the returned list together with its
    output and the token positions afterwards: lets a test replay the same inputs through another
    implementation and compare call by call."""
    log: List[ForwardInputOutput] = []
    inner = cache.forward

    def wrapped(query, key, value, token_idx):
        pos = cache.input_pos
        out = inner(query, key, value, token_idx)
        cpu = lambda t: None if t is None else t.detach().to("cpu").clone()  # noqa: E731
        tp = cache.token_positions() if hasattr(cache, "token_positions") and cache.current_length > 0 else None
        log.append(ForwardInputOutput(ForwardInput(cpu(query), cpu(key), cpu(value), cpu(token_idx), pos), cpu(out), cpu(tp)))
        return out

    cache.forward = wrapped
    return log


# ---------------------------------------------------------------------------------------------------
# Before / after snapshots: freeze what a cache does today, check a changed implementation against it
# (role of ``keys_values/kvcache/test_before_after.py:142-343``)
# ---------------------------------------------------------------------------------------------------
def _cache_state(cache: KVCache) -> Dict[str, torch.Tensor]:
    """What defines a cache after a call: keys and values as attention sees them, token positions, and the
    scores of score-based policies."""
    state: Dict[str, torch.Tensor] = {}
    if cache.current_length > 0:
        kv = cache.get_keys_values()
        if kv is not None:
            state["keys"], state["values"] = kv.keys().detach().float().cpu(), kv.values().detach().float().cpu()
        if hasattr(cache, "token_positions"):
            state["token_positions"] = cache.token_positions().detach().cpu()
    scores = getattr(cache, "scores", None)
    if torch.is_tensor(scores):
        state["scores"] = scores.detach().float().cpu()
    return state


class ForwardSnapshots:
    """``ForwardSnapshots(cache, path_mask, num_steps).store()`` writes one file per ``forward`` call
    (``path_mask.format(k)``: inputs, output, state afterwards). With a changed implementation,
    ``.compare(**tolerances)`` feeds every call the STORED inputs (so that small differences do not drift from
    call to call into different eviction decisions) and checks output and state against the files; the indices
    of the calls that were compared are in ``.compared``."""

    def __init__(self, cache: KVCache, path_mask: str, num_steps: int):
        self.cache, self.path_mask, self.num_steps = cache, path_mask, num_steps
        self.compared: List[int] = []
        self._inner = cache.forward
        self._k = 0

    def _restore(self) -> None:
        self.cache.forward = self._inner

    def store(self) -> "ForwardSnapshots":
        def wrapped(query, key, value, token_idx):
            pos = self.cache.input_pos
            out = self._inner(query, key, value, token_idx)
            if self._k < self.num_steps:
                cpu = lambda t: None if t is None else t.detach().cpu().clone()  # noqa: E731
                torch.save({"inputs": dict(query=cpu(query), key=cpu(key), value=cpu(value), token_idx=cpu(token_idx), input_pos=pos),
                            "output": cpu(out).float(), "state": _cache_state(self.cache)}, self.path_mask.format(self._k))
            self._k += 1
            return out

        self.cache.forward = wrapped
        return self

    def compare(self, **tol) -> "ForwardSnapshots":
        tol = tol or dict(atol=1e-5, rtol=1e-5)

        def wrapped(query, key, value, token_idx):
            if self._k >= self.num_steps:
                self._k += 1
                return self._inner(query, key, value, token_idx)
            rec = torch.load(self.path_mask.format(self._k), weights_only=False)
            inp = rec["inputs"]
            if inp["input_pos"] != self.cache.input_pos:
                raise AssertionError(f"call {self._k}: input_pos {self.cache.input_pos}, snapshot has {inp['input_pos']}")
            to = lambda t, like: None if t is None else t.to(device=like.device, dtype=like.dtype)  # noqa: E731
            out = self._inner(to(inp["query"], query), to(inp["key"], key), to(inp["value"], value),
                              None if token_idx is None else to(inp["token_idx"], token_idx))
            torch.testing.assert_close(out.detach().float().cpu(), rec["output"], msg=lambda m: f"call {self._k}, output: {m}", **tol)
            now = _cache_state(self.cache)
            for name, want in rec["state"].items():
                if name == "token_positions":
                    assert torch.equal(now[name], want), f"call {self._k}: token positions differ"
                else:
                    torch.testing.assert_close(now[name], want, msg=lambda m, n=name: f"call {self._k}, {n}: {m}", **tol)
            self.compared.append(self._k)
            self._k += 1
            return out

        self.cache.forward = wrapped
        return self

    def stop(self) -> None:
        self._restore()
