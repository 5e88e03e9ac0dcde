"""Model configuration.

A self-contained dataclass that uses the LitGPT field names, so that a
``model_config.yaml`` written next to a ``lit_model.pth`` loads unchanged
(parity: ``keys_values/config.py:23-43`` and the LitGPT ``Config`` it extends;
field list as in ``keys_values/scripts/convert_lora_to_litgpt/model_config.yaml``).
A small registry of named architectures replaces LitGPT's ``name_to_config``.
"""
from __future__ import annotations

import copy
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, List, Optional, Type, Union

import yaml


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of ``k`` that is ``>= n``."""
    if n % k == 0:
        return n
    return n + k - (n % k)


@dataclass
class Config:
    name: str = ""
    hf_config: dict = field(default_factory=dict)
    # General size parameters
    block_size: int = 4096
    n_layer: int = 16
    n_embd: int = 4096
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    # Transformer block (structure, normalizations)
    norm_class_name: str = "LayerNorm"
    norm_eps: float = 1e-5
    norm_qk: bool = False
    norm_qk_type: str = "default"
    post_attention_norm: bool = False
    post_mlp_norm: bool = False
    parallel_residual: bool = True
    shared_attention_norm: bool = False
    norm_1: bool = True
    norm_2: bool = True
    # Transformer block (self-attention)
    n_head: int = 32
    head_size: Optional[int] = None
    n_query_groups: Optional[int] = None
    attn_bias: bool = False
    attention_scores_scalar: Optional[int] = None
    sliding_window_size: Optional[int] = None
    sliding_window_indices: Optional[List[int]] = None
    attention_logit_softcapping: Optional[float] = None
    latent_attention: Optional[dict] = None
    # Rotary position embedding
    rope_base: int = 10000
    rotary_percentage: float = 0.25
    rope_condense_ratio: int = 1
    rope_adjustments: Optional[dict] = None
    rope_local_base_freq: Optional[float] = None
    rope_indices: Optional[List[int]] = None
    # Transformer block (MLP)
    intermediate_size: Optional[int] = None
    moe_intermediate_size: Optional[int] = None
    bias: bool = True
    mlp_class_name: str = "GptNeoxMLP"
    gelu_approximate: str = "none"
    n_expert: int = 0
    n_shared_expert: Optional[int] = None
    n_expert_groups: Optional[int] = None
    n_topk_groups: Optional[int] = None
    n_topk_scores_per_group: Optional[int] = None
    n_expert_per_token: int = 0
    first_k_dense_replace: Optional[int] = None
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = False
    # GPT before/after blocks
    scale_embeddings: bool = False
    lm_head_bias: bool = False
    final_logit_softcapping: Optional[float] = None
    # Added by keys_values (config.py:26-30): use the in-repo RMSNorm
    own_rms_norm_implementation: bool = True

    def __post_init__(self):
        if not self.name:
            self.name = self.hf_config.get("name", self.name)
        if self.head_size is None:
            assert self.n_embd % self.n_head == 0
            self.head_size = self.n_embd // self.n_head
        if self.padded_vocab_size is None:
            self.padded_vocab_size = find_multiple(self.vocab_size, self.padding_multiple)
        else:
            self.vocab_size = min(self.vocab_size, self.padded_vocab_size)
        if self.n_query_groups is not None:
            assert self.n_head % self.n_query_groups == 0
        else:
            self.n_query_groups = self.n_head
        if self.intermediate_size is None:
            if self.mlp_class_name == "LLaMAMLP":
                raise ValueError(f"The config {self.name!r} needs to set `intermediate_size`")
            self.intermediate_size = 4 * self.n_embd
        self.rope_n_elem = int(self.rotary_percentage * self.head_size)
        if self.sliding_window_size is not None and self.sliding_window_indices is None:
            self.sliding_window_indices = [1] * self.n_layer
        if self.rope_local_base_freq is not None and self.rope_indices is None:
            self.rope_indices = [1] * self.n_layer

    # ----------------------------------------------------------- construction
    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "Config":
        if name not in name_to_config:
            raise ValueError(f"{name!r} is not a supported config name; known: {sorted(name_to_config)}")
        conf = copy.deepcopy(name_to_config[name])
        conf.update(kwargs)
        return cls(**conf)

    @classmethod
    def from_file(cls, path: Union[str, Path], **kwargs: Any) -> "Config":
        with open(path, encoding="utf-8") as fp:
            file_kwargs = yaml.safe_load(fp)
            if file_kwargs is None:
                raise ValueError(f"{path} is empty which is likely unexpected.")
        file_kwargs.update(kwargs)
        known = {f.name for f in fields(cls)}
        file_kwargs = {k: v for k, v in file_kwargs.items() if k in known}
        return cls(**file_kwargs)

    @classmethod
    def from_checkpoint(cls, path: Union[str, Path], **kwargs: Any) -> "Config":
        """``path`` is a checkpoint directory holding ``model_config.yaml``."""
        path = Path(path)
        if (config_path := path / "model_config.yaml").is_file():
            return cls.from_file(config_path, **kwargs)
        if (model_name := path.name) in name_to_config:
            return cls.from_name(model_name, **kwargs)
        raise FileNotFoundError(f"For {str(path)!r} neither 'model_config.yaml' nor matching config exists.")

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        return d

    def save(self, path: Union[str, Path]) -> None:
        with open(path, "w", encoding="utf-8") as fp:
            yaml.safe_dump(self.to_dict(), fp)

    # ------------------------------------------------------------- factories
    @property
    def mlp_class(self) -> Type:
        from keys_values_b200.models import model as _m

        return getattr(_m, self.mlp_class_name)

    @property
    def norm_class(self) -> Type:
        """Normalization layer constructor (parity: ``keys_values/config.py:32-43``).

        ``RMSNorm`` maps to the in-repo implementation (Gemma configs get
        ``add_unit_offset=True``); any other name is taken from ``torch.nn``.
        """
        from functools import partial

        import torch

        from keys_values_b200.models.model import RMSNorm

        if self.norm_class_name == "RMSNorm":
            return partial(RMSNorm, add_unit_offset="Gemma" in self.name)
        if self.norm_class_name == "LayerNorm" and "OLMo" in self.name:
            return partial(torch.nn.LayerNorm, elementwise_affine=False)
        return getattr(torch.nn, self.norm_class_name)


# --------------------------------------------------------------------------
# Registry of named architectures. Only architecture hyper-parameters live here:
# weights come from a ``lit_model.pth`` or from random initialisation.
# --------------------------------------------------------------------------
_llama_like = dict(
    rotary_percentage=1.0,
    parallel_residual=False,
    bias=False,
    norm_class_name="RMSNorm",
    mlp_class_name="LLaMAMLP",
)

configs: List[dict] = [
    # Tiny test models
    dict(
        name="tiny-gpt",
        block_size=1024, vocab_size=512, padded_vocab_size=512, n_layer=2, n_embd=64,
        n_head=4, n_query_groups=2, head_size=16, intermediate_size=172,
        norm_eps=1e-5, rope_base=10000, **_llama_like,
    ),
    dict(
        name="tiny-qwen3",
        block_size=4096, vocab_size=1024, padded_vocab_size=1024, n_layer=2, n_embd=256,
        n_head=8, n_query_groups=2, head_size=128, intermediate_size=512, norm_qk=True,
        norm_eps=1e-6, rope_base=1000000, **_llama_like,
    ),
    dict(  # head size 64 (Llama-3.2-1B, Qwen2.5-0.5B shapes)
        name="tiny-llama-d64",
        block_size=4096, vocab_size=1024, padded_vocab_size=1024, n_layer=2, n_embd=256,
        n_head=4, n_query_groups=2, head_size=64, intermediate_size=512,
        norm_eps=1e-5, rope_base=500000, **_llama_like,
    ),
    dict(  # head size 256 with a window layer and capped scores (Gemma-2 2b / 9b shapes): forward kernels only
        name="tiny-gemma2-d256",
        block_size=4096, vocab_size=1024, padded_vocab_size=1024, n_layer=2, n_embd=256,
        n_head=4, n_query_groups=2, head_size=256, intermediate_size=512, norm_eps=1e-6,
        rotary_percentage=1.0, parallel_residual=False, bias=False, norm_class_name="RMSNorm",
        mlp_class_name="GemmaMLP", gelu_approximate="tanh", scale_embeddings=True,
        post_attention_norm=True, post_mlp_norm=True, sliding_window_size=96, sliding_window_indices=[1, 0],
        attention_logit_softcapping=4.0, final_logit_softcapping=30.0,
    ),
    dict(  # Gemma-2 style: every other layer with a sliding window, capped attention scores and logits
        name="tiny-gemma2",
        block_size=4096, vocab_size=1024, padded_vocab_size=1024, n_layer=2, n_embd=256,
        n_head=8, n_query_groups=2, head_size=128, intermediate_size=512, norm_eps=1e-6,
        rotary_percentage=1.0, parallel_residual=False, bias=False, norm_class_name="RMSNorm",
        mlp_class_name="GemmaMLP", gelu_approximate="tanh", scale_embeddings=True,
        post_attention_norm=True, post_mlp_norm=True, sliding_window_size=96, sliding_window_indices=[1, 0],
        attention_logit_softcapping=4.0, final_logit_softcapping=30.0,
    ),
    dict(
        name="pythia-14m",
        block_size=512, n_layer=6, n_embd=128, n_head=4, padding_multiple=128,
    ),
    # Qwen 2.5
    dict(
        name="Qwen2.5-0.5B", hf_config=dict(org="Qwen", name="Qwen2.5-0.5B"),
        block_size=32768, vocab_size=151643, padded_vocab_size=151936, n_layer=24, n_head=14,
        n_embd=896, n_query_groups=2, attn_bias=True, intermediate_size=4864, norm_eps=1e-6,
        rope_base=1000000, **_llama_like,
    ),
    dict(
        name="Qwen2.5-1.5B", hf_config=dict(org="Qwen", name="Qwen2.5-1.5B"),
        block_size=131072, vocab_size=151643, padded_vocab_size=151936, n_layer=28, n_head=12,
        n_embd=1536, n_query_groups=2, attn_bias=True, intermediate_size=8960, norm_eps=1e-6,
        rope_base=1000000, **_llama_like,
    ),
    dict(
        name="Qwen2.5-7B", hf_config=dict(org="Qwen", name="Qwen2.5-7B"),
        block_size=131072, vocab_size=151643, padded_vocab_size=152064, n_layer=28, n_head=28,
        n_embd=3584, n_query_groups=4, attn_bias=True, intermediate_size=18944, norm_eps=1e-6,
        rope_base=1000000, **_llama_like,
    ),
    # Qwen 3
    dict(
        name="Qwen3-0.6B", hf_config=dict(org="Qwen", name="Qwen3-0.6B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=28, n_head=16,
        n_embd=1024, n_query_groups=8, head_size=128, intermediate_size=3072, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-1.7B", hf_config=dict(org="Qwen", name="Qwen3-1.7B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=28, n_head=16,
        n_embd=2048, n_query_groups=8, head_size=128, intermediate_size=6144, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-4B", hf_config=dict(org="Qwen", name="Qwen3-4B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=36, n_head=32,
        n_embd=2560, n_query_groups=8, head_size=128, intermediate_size=9728, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-4B-Instruct-2507", hf_config=dict(org="Qwen", name="Qwen3-4B-Instruct-2507"),
        block_size=262144, vocab_size=151643, padded_vocab_size=151936, n_layer=36, n_head=32,
        n_embd=2560, n_query_groups=8, head_size=128, intermediate_size=9728, norm_eps=1e-6,
        rope_base=5000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-8B", hf_config=dict(org="Qwen", name="Qwen3-8B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=36, n_head=32,
        n_embd=4096, n_query_groups=8, head_size=128, intermediate_size=12288, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-14B", hf_config=dict(org="Qwen", name="Qwen3-14B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=40, n_head=40,
        n_embd=5120, n_query_groups=8, head_size=128, intermediate_size=17408, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    dict(
        name="Qwen3-32B", hf_config=dict(org="Qwen", name="Qwen3-32B"),
        block_size=40960, vocab_size=151643, padded_vocab_size=151936, n_layer=64, n_head=64,
        n_embd=5120, n_query_groups=8, head_size=128, intermediate_size=25600, norm_eps=1e-6,
        rope_base=1000000, norm_qk=True, **_llama_like,
    ),
    # Llama 3.x
    dict(
        name="Llama-3-8B", hf_config=dict(org="meta-llama", name="Meta-Llama-3-8B"),
        block_size=8192, vocab_size=128000, padded_vocab_size=128256, n_layer=32, n_head=32,
        n_embd=4096, n_query_groups=8, intermediate_size=14336, norm_eps=1e-5, rope_base=500000,
        **_llama_like,
    ),
    dict(
        name="Llama-3.1-8B", hf_config=dict(org="meta-llama", name="Meta-Llama-3.1-8B"),
        block_size=131072, vocab_size=128000, padded_vocab_size=128256, n_layer=32, n_head=32,
        n_embd=4096, n_query_groups=8, intermediate_size=14336, norm_eps=1e-5, rope_base=500000,
        rope_adjustments=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_seq_len=8192),
        **_llama_like,
    ),
    dict(
        name="Llama-3.2-1B", hf_config=dict(org="meta-llama", name="Llama-3.2-1B"),
        block_size=131072, vocab_size=128000, padded_vocab_size=128256, n_layer=16, n_head=32,
        n_embd=2048, n_query_groups=8, intermediate_size=8192, norm_eps=1e-5, rope_base=500000,
        rope_adjustments=dict(factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_seq_len=8192),
        **_llama_like,
    ),
    # Gemma 2 (softcapping, sliding window, post norms, GemmaMLP)
    dict(
        name="Gemma-2-2b", hf_config=dict(org="google", name="gemma-2-2b"),
        block_size=8192, vocab_size=256000, padded_vocab_size=256000, n_layer=26, n_head=8,
        n_embd=2304, n_query_groups=4, head_size=256, intermediate_size=9216, norm_eps=1e-6,
        rotary_percentage=1.0, parallel_residual=False, bias=False, norm_class_name="RMSNorm",
        mlp_class_name="GemmaMLP", gelu_approximate="tanh", scale_embeddings=True,
        post_attention_norm=True, post_mlp_norm=True, sliding_window_size=4096,
        sliding_window_indices=[1 if i % 2 == 0 else 0 for i in range(26)],
        attention_scores_scalar=256, attention_logit_softcapping=50.0, final_logit_softcapping=30.0,
    ),
    # Mistral-style with sliding window
    dict(
        name="Mistral-7B-v0.1", hf_config=dict(org="mistralai", name="Mistral-7B-v0.1"),
        block_size=4096, vocab_size=32000, padded_vocab_size=32000, n_layer=32, n_head=32, n_embd=4096,
        n_query_groups=8, intermediate_size=14336, norm_eps=1e-5, sliding_window_size=4096,
        **_llama_like,
    ),
    # Phi-like parallel residual with partial rotary and LayerNorm
    dict(
        name="phi-2", hf_config=dict(org="microsoft", name="phi-2"),
        block_size=2048, vocab_size=50257, padded_vocab_size=51200, n_layer=32, n_head=32, n_embd=2560,
        rotary_percentage=0.4, shared_attention_norm=True, lm_head_bias=True, gelu_approximate="tanh",
    ),
]

name_to_config: Dict[str, dict] = {c["name"]: c for c in configs}
