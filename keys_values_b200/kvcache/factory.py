"""Creation of KV caches by name (``keys_values/kvcache/factory.py:50-598``).

Names are ``<policy>-<buffers>`` with policy in ``dense, lastrec, smart-lastrec,
h2o, h2o-vlen, qh2o, qh2o-vlen, h2o-orig`` and buffers in ``default,
torch-quantized4, torch-quantized8, bnb-quantized4, bnb-quantized8``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union


from keys_values_b200.config import Config
from keys_values_b200.kvcache.base import KVCache, KVCacheParams
from keys_values_b200.kvcache.basics import DenseKVCache, LastRecentlyInsertedKVCache
from keys_values_b200.kvcache.buffers import DefaultKVCacheBuffers
from keys_values_b200.kvcache.consts import SUPPORTED_QUANTIZERS, split_name
from keys_values_b200.kvcache.h2o import H2OKVCache, H2OOriginalKVCache, VLengthH2OKVCache
from keys_values_b200.kvcache.qh2o import QuantizedH2OKVCache, QuantizedVLengthH2OKVCache
from keys_values_b200.kvcache.quant_buffers import (
    DequantizedKVCacheBuffers,
    QuantizedKVCacheBuffers,
    create_quantized_kv_buffers,
    get_quant_kwargs,
)
from keys_values_b200.kvcache.smart_lastrec import SmartInitialLastRecentlyInsertedKVCache

_POLICIES = {
    "dense": DenseKVCache,
    "lastrec": LastRecentlyInsertedKVCache,
    "smart-lastrec": SmartInitialLastRecentlyInsertedKVCache,
    "h2o": H2OKVCache,
    "h2o-vlen": VLengthH2OKVCache,
    "qh2o": QuantizedH2OKVCache,
    "qh2o-vlen": QuantizedVLengthH2OKVCache,
    "h2o-orig": H2OOriginalKVCache,
}

SUPPORTED_CACHES: Dict[str, type] = {
    f"{p}-{q}": cls
    for p, cls in _POLICIES.items()
    for q in SUPPORTED_QUANTIZERS
    if not (p.startswith("qh2o") and q == "default")
}


class KVCacheFactory:
    @staticmethod
    def supported_names() -> List[str]:
        return list(SUPPORTED_CACHES.keys())

    @staticmethod
    def needs_attn_weights(name: str) -> bool:
        return issubclass(KVCacheFactory._cache_type(name), (H2OKVCache, H2OOriginalKVCache))

    @staticmethod
    def _cache_type(name: str) -> type:
        cache_type = SUPPORTED_CACHES.get(name)
        if cache_type is None:
            if name in ("qh2o-default", "qh2o-vlen-default"):
                raise ValueError(f"{name[:-8]} can only be used with quantized buffers")
            raise ValueError(f"name = {name} not supported")
        return cache_type

    @staticmethod
    def create_single(
        name: str,
        config: Config,
        max_batch_size: int,
        cache_length: int,
        block_idx: int,
        device=None,
        dtype=None,
        cache_kwargs: Optional[Dict[str, Any]] = None,
    ) -> KVCache:
        model_like = type("_M", (), {"config": config, "mha": None})()
        return KVCacheFactory._create(model_like, name, max_batch_size, [cache_length], block_idx, block_idx + 1, device, dtype, cache_kwargs)[0]

    @staticmethod
    def create(
        gpt_model,
        name: str,
        max_batch_size: int,
        cache_length: Union[int, List[int]],
        start: int = 0,
        end: Optional[int] = None,
        device=None,
        dtype=None,
        cache_kwargs: Optional[Dict[str, Any]] = None,
    ) -> List[KVCache]:
        """One cache per layer in ``range(start, end)``; quantized buffers of layers
        with the same cache length share one de-quantization scratch. The caches
        use the position encoding / SDPA settings of ``gpt_model``."""
        config = gpt_model.config
        if end is None:
            end = config.n_layer
        if not (0 <= start < end <= config.n_layer):
            raise ValueError(f"start={start}, end={end}, must be 0 <= start < end <= {config.n_layer}")
        num_layers = end - start
        if not isinstance(cache_length, (list, tuple)):
            cache_length = [cache_length] * num_layers
        elif len(cache_length) == 1:
            cache_length = [cache_length[0]] * num_layers
        elif len(cache_length) != num_layers:
            raise ValueError(f"len(cache_length) = {len(cache_length)}, must be 1 or {num_layers}")
        if not all(x > 0 for x in cache_length):
            raise ValueError(f"cache_length = {cache_length}, must contain only positive integers")
        return KVCacheFactory._create(gpt_model, name, max_batch_size, list(cache_length), start, end, device, dtype, cache_kwargs)

    @staticmethod
    def _create(gpt_model, name, max_batch_size, cache_lengths, start, end, device, dtype, cache_kwargs) -> List[KVCache]:
        config = gpt_model.config
        cache_type = KVCacheFactory._cache_type(name)
        cache_kwargs = dict(cache_kwargs or {})
        max_num_ranges = cache_kwargs.pop("max_num_ranges", None)
        allocate_buffers = cache_kwargs.pop("allocate_buffers", False)
        mha = getattr(gpt_model, "mha", None)
        if mha is not None:
            cache_kwargs.setdefault("mha", mha)
        _, qname = split_name(name)
        if qname == "default":
            cache_kwargs.pop("blocks_over_heads", None)
            return [
                cache_type.from_config(
                    config=config, max_batch_size=max_batch_size, cache_length=c_len,
                    block_idx=start + i, device=device, dtype=dtype, **cache_kwargs,
                )
                for i, c_len in enumerate(cache_lengths)
            ]
        if dtype is None:
            raise ValueError(f"dtype must be given for quantized cache buffers ({qname})")
        params = KVCacheParams(max_batch_size, config.n_query_groups, cache_lengths[0], config.head_size, config.n_head, dtype)
        _, _, policy_kwargs = get_quant_kwargs(params, qname, cache_kwargs)
        buffers = create_quantized_kv_buffers(
            qname=qname, cache_lengths=cache_lengths, cache_params=params, cache_kwargs=cache_kwargs,
            dequant_kwargs=dict(max_num_ranges=max_num_ranges), allocate_buffers=allocate_buffers,
            device=device, first_block_idx=start,
        )
        return [cache_type(config=config, buffers=b, block_idx=start + i, **policy_kwargs) for i, b in enumerate(buffers)]

    @staticmethod
    def create_cpu_offloading(
        gpt_model,
        name: str,
        max_batch_size: int,
        cache_length: int,
        device=None,
        dtype=None,
        cache_kwargs: Optional[Dict[str, Any]] = None,
        pin_memory: bool = True,
    ):
        """Caches whose quantized storage lives in (pinned) host memory, except for
        the layer being processed. Returns ``(kv_caches, offloader)``."""
        from keys_values_b200.kvcache.offloading import KVCacheOffloader

        _, qname = split_name(name)
        if qname == "default":
            raise ValueError("CPU offloading needs quantized buffers")
        caches = KVCacheFactory.create(gpt_model, name, max_batch_size, cache_length, device=device, dtype=dtype, cache_kwargs=cache_kwargs)
        offloader = KVCacheOffloader([c.kv_buffers for c in caches], pin_memory=pin_memory)
        return caches, offloader

    @staticmethod
    def size_estimate(kv_caches: List[KVCache]) -> Tuple[int, Dict[str, int]]:
        total, detail = 0, {}
        seen_scratch = set()
        for c in kv_caches:
            sz, d = c.size_estimate()
            total += sz
            for k, v in d.items():
                detail[k] = detail.get(k, 0) + v
            dq = getattr(getattr(c, "kv_buffers", None), "dequant_buffers", None)
            if dq is not None and id(dq) not in seen_scratch:
                seen_scratch.add(id(dq))
                s, _ = dq.size_estimate()
                total += s
                detail["dequant_buffers"] = detail.get("dequant_buffers", 0) + s
        return total, detail

    @staticmethod
    def size_estimate_apriori(name: str, config: Config, max_batch_size: int, cache_length: int, n_layer: Optional[int] = None, dtype=None, **kwargs):
        cache_type = KVCacheFactory._cache_type(name)
        _, qname = split_name(name)
        n_layer = config.n_layer if n_layer is None else n_layer
        params = KVCacheParams(max_batch_size, config.n_query_groups, cache_length, config.head_size, config.n_head, dtype)
        sz, d = cache_type.size_estimate_apriori(params, **kwargs)
        if qname != "default":
            raw, _ = DefaultKVCacheBuffers.size_estimate_apriori(params)
            qs, _ = QuantizedKVCacheBuffers.size_estimate_apriori(params, num_bits=int(qname[-1]))
            sz = sz - raw + qs
            return n_layer * sz + raw, dict(d, dequant_buffers=raw)
        return n_layer * sz, d


def deallocate_kv_cache_buffers(kv_caches: List[Optional[KVCache]]) -> None:
    for c in kv_caches:
        if c is not None and hasattr(c, "deallocate_buffers"):
            c.deallocate_buffers()
            dq = getattr(c.kv_buffers, "dequant_buffers", None)
            if dq is not None:
                dq.deallocate()


def deallocate_kv_cache_buffers_of_model(gpt_model) -> None:
    deallocate_kv_cache_buffers(gpt_model.get_kv_caches())


def cleanup_cache_kwargs(name: str, cache_kwargs: Dict[str, Any]) -> Dict[str, Any]:
    """Remove entries from ``cache_kwargs`` that the cache named ``name`` does not take."""
    cname, qname = split_name(name)
    allowed = {"mha", "tmp_array_limit_gb"}
    if qname != "default":
        allowed |= {"blocks_over_heads", "max_num_ranges", "allocate_buffers"}
    if cname in ("lastrec",):
        allowed |= {"init_grace_tokens"}
    if cname == "smart-lastrec":
        allowed |= {"tokenizer", "end_initial_regex", "max_initial_fraction", "include_end_string", "pad_id"}
    if "h2o" in cname:
        allowed |= {"grace_period", "replay_log_blocksize", "detach_attn_weights", "keep_initial_fraction", "max_chunk_size"}
        if cname != "h2o-orig":
            allowed |= {"normalize_scores"}
    if cname.startswith("qh2o"):
        allowed |= {"combination_constant", "scratch_blocksize"}
    return {k: v for k, v in cache_kwargs.items() if k in allowed}
