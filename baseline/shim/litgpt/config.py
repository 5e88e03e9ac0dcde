"""Stand-in for ``litgpt.config``: the model configuration dataclass with LitGPT's field names."""
from __future__ import annotations

from copy import deepcopy
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, List, Literal, Optional, Type, Union

import torch
import yaml


def find_multiple(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class Config:
    name: str = ""
    hf_config: dict = field(default_factory=dict)
    block_size: int = 4096
    n_layer: int = 16
    n_embd: int = 4096
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    norm_class_name: Literal["LayerNorm", "RMSNorm"] = "LayerNorm"
    norm_eps: float = 1e-5
    norm_qk: bool = False
    norm_qk_type: Literal["default", "olmo2"] = "default"
    post_attention_norm: bool = False
    post_mlp_norm: bool = False
    parallel_residual: bool = True
    shared_attention_norm: bool = False
    norm_1: bool = True
    norm_2: bool = True
    n_head: int = 32
    head_size: Optional[int] = None
    n_query_groups: Optional[int] = None
    attn_bias: bool = False
    attention_scores_scalar: Optional[int] = None
    sliding_window_size: Optional[int] = None
    sliding_window_indices: Optional[List] = None
    attention_logit_softcapping: Optional[float] = None
    latent_attention: Optional[dict] = None
    rope_base: int = 10000
    rotary_percentage: float = 0.25
    rope_condense_ratio: int = 1
    rope_adjustments: Optional[dict] = None
    rope_local_base_freq: Optional[float] = None
    rope_indices: Optional[List] = None
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
    scale_embeddings: bool = False
    lm_head_bias: bool = False
    final_logit_softcapping: Optional[float] = None

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
                raise ValueError(f"The config {self.name!r} needs to set the `intermediate_size`")
            self.intermediate_size = 4 * self.n_embd
        self.rope_n_elem = int(self.rotary_percentage * self.head_size)
        if self.sliding_window_size is not None and self.sliding_window_indices is None:
            self.sliding_window_indices = [1] * self.n_layer
        if self.rope_local_base_freq is not None and self.rope_indices is None:
            self.rope_indices = [1] * self.n_layer

    @classmethod
    def from_name(cls, name: str, **kwargs: Any):
        if name not in name_to_config:
            raise ValueError(f"{name!r} is not a supported config name")
        conf = deepcopy(name_to_config[name])
        conf.update(kwargs)
        return cls(**conf)

    @classmethod
    def from_file(cls, path: Union[str, Path], **kwargs: Any):
        with open(path, encoding="utf-8") as fp:
            file_kwargs = yaml.safe_load(fp)
        if file_kwargs is None:
            raise ValueError(f"{path} is empty which is likely unexpected.")
        file_kwargs.update(kwargs)
        return cls(**file_kwargs)

    @classmethod
    def from_checkpoint(cls, path: Path, **kwargs: Any):
        if (config_path := path / "model_config.yaml").is_file():
            return cls.from_file(config_path, **kwargs)
        if (model_name := path.name) in name_to_config:
            return cls.from_name(model_name, **kwargs)
        raise FileNotFoundError(f"For {str(path)!r} neither 'model_config.yaml' nor matching config exists.")

    @property
    def mlp_class(self) -> Type:
        import litgpt.model

        return getattr(litgpt.model, self.mlp_class_name)

    @property
    def norm_class(self) -> Type:
        if self.norm_class_name == "RMSNorm":
            from functools import partial

            from litgpt.model import RMSNorm

            return partial(RMSNorm, add_unit_offset="Gemma" in self.name)
        return getattr(torch.nn, self.norm_class_name)


def _qwen3(name, n_layer, n_embd, n_head, inter, block=40960):
    return dict(
        name=name, hf_config=dict(org="Qwen", name=name), block_size=block, vocab_size=151643, padded_vocab_size=151936,
        n_layer=n_layer, n_head=n_head, n_embd=n_embd, n_query_groups=8, head_size=128, rotary_percentage=1.0,
        parallel_residual=False, bias=False, norm_class_name="RMSNorm", mlp_class_name="LLaMAMLP",
        intermediate_size=inter, norm_eps=1e-6, rope_base=1000000, norm_qk=True,
    )


name_to_config = {
    "Qwen3-4B": _qwen3("Qwen3-4B", 36, 2560, 32, 9728),
    "Qwen3-4B-Instruct-2507": dict(_qwen3("Qwen3-4B-Instruct-2507", 36, 2560, 32, 9728, block=262144), rope_base=5000000),
    "Qwen3-14B": _qwen3("Qwen3-14B", 40, 5120, 40, 17408),
    "Llama-3-8B": dict(
        name="Llama-3-8B", hf_config=dict(org="meta-llama", name="Meta-Llama-3-8B"), block_size=8192, vocab_size=128000,
        padded_vocab_size=128256, n_layer=32, n_head=32, n_embd=4096, n_query_groups=8, rotary_percentage=1.0,
        parallel_residual=False, bias=False, norm_class_name="RMSNorm", mlp_class_name="LLaMAMLP",
        intermediate_size=14336, rope_base=500000,
    ),
}
configs = list(name_to_config.values())
