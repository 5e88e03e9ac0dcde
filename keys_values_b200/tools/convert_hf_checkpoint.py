"""Converts a Hugging Face checkpoint of a Llama-like decoder (Llama 2/3, Mistral, Qwen2.5, Qwen3,
Gemma 2) into this framework's checkpoint directory (``lit_model.pth`` + ``model_config.yaml``, the
LitGPT layout that ``keys_values`` reads).

    python -m keys_values_b200.tools.convert_hf_checkpoint <hf_dir> <out_dir> [--model-name Qwen3-4B]

The weights may be ``*.safetensors`` or ``pytorch_model*.bin`` shards. Only the parameter names are
mapped and ``q | k | v`` are concatenated into one matrix; no value is changed (both sides use the
"rotate half" RoPE convention). Role of ``litgpt/scripts/convert_hf_checkpoint.py``, which the
reference relies on through ``litgpt download`` (``keys_values/finetune/longcontext_full.py:356-389``).
"""
from __future__ import annotations

import argparse
import json
import re
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

import torch

from keys_values_b200.config import Config

_LAYER = re.compile(r"^model\.layers\.(\d+)\.(.+)$")

_PER_LAYER = {
    "input_layernorm.weight": "norm_1.weight",
    "post_attention_layernorm.weight": "norm_2.weight",
    "self_attn.o_proj.weight": "attn.proj.weight",
    "self_attn.o_proj.bias": "attn.proj.bias",
    "self_attn.q_norm.weight": "attn.norm_q.weight",
    "self_attn.k_norm.weight": "attn.norm_k.weight",
    "mlp.gate_proj.weight": "mlp.fc_1.weight",
    "mlp.up_proj.weight": "mlp.fc_2.weight",
    "mlp.down_proj.weight": "mlp.proj.weight",
    # Gemma 2: norms around attention and MLP
    "pre_feedforward_layernorm.weight": "norm_2.weight",
    "post_feedforward_layernorm.weight": "post_mlp_norm.weight",
}
_GLOBAL = {
    "model.embed_tokens.weight": "transformer.wte.weight",
    "model.norm.weight": "transformer.ln_f.weight",
    "lm_head.weight": "lm_head.weight",
}


def convert_state_dict(hf_sd: Dict[str, torch.Tensor], config: Config) -> Dict[str, torch.Tensor]:
    """HF names -> this framework's names. ``hf_sd`` may be a lazily loading mapping."""
    out: Dict[str, torch.Tensor] = {}
    qkv: Dict[Tuple[int, str, str], torch.Tensor] = {}
    gemma2 = bool(getattr(config, "post_attention_norm", False))
    for name in list(hf_sd.keys()):
        t = hf_sd[name]
        if name in _GLOBAL:
            out[_GLOBAL[name]] = t
            continue
        m = _LAYER.match(name)
        if m is None:
            if name.endswith("rotary_emb.inv_freq"):
                continue
            raise KeyError(f"unexpected parameter {name}")
        i, rest = int(m.group(1)), m.group(2)
        q = re.match(r"^self_attn\.([qkv])_proj\.(weight|bias)$", rest)
        if q is not None:
            qkv[(i, q.group(1), q.group(2))] = t
            continue
        if gemma2 and rest == "post_attention_layernorm.weight":
            out[f"transformer.h.{i}.post_attention_norm.weight"] = t
            continue
        if rest not in _PER_LAYER:
            if rest.endswith("rotary_emb.inv_freq"):
                continue
            raise KeyError(f"unexpected parameter {name}")
        out[f"transformer.h.{i}.{_PER_LAYER[rest]}"] = t
    for i in range(config.n_layer):
        for kind in ("weight", "bias"):
            parts = [qkv.get((i, c, kind)) for c in "qkv"]
            if all(p is None for p in parts):
                continue
            if any(p is None for p in parts):
                raise KeyError(f"layer {i}: incomplete q/k/v {kind}")
            out[f"transformer.h.{i}.attn.qkv.{kind}"] = torch.cat(parts, dim=0)
    if "lm_head.weight" not in out:  # tied embeddings
        out["lm_head.weight"] = out["transformer.wte.weight"]
    return out


def _rope_theta(hf: dict) -> float:
    """``rope_theta`` sits at the top level of older ``config.json`` files and inside
    ``rope_parameters`` (or ``rope_scaling``) of newer ones."""
    for holder in (hf, hf.get("rope_parameters") or {}, hf.get("rope_scaling") or {}):
        if holder.get("rope_theta") is not None:
            return float(holder["rope_theta"])
    return 10000.0


def config_from_hf(hf: dict, name: Optional[str] = None) -> Config:
    """A :class:`Config` from a HF ``config.json`` dictionary (a registry entry if ``name`` is known)."""
    if name is not None:
        return Config.from_name(name)
    arch = ((hf.get("architectures") or [""])[0] + " " + str(hf.get("model_type", ""))).lower()
    n_head = hf["num_attention_heads"]
    head_size = hf.get("head_dim") or hf["hidden_size"] // n_head
    kw = dict(
        name=hf.get("_name_or_path") or arch.strip() or "hf-model", block_size=hf.get("max_position_embeddings", 4096),
        vocab_size=hf["vocab_size"], padded_vocab_size=hf["vocab_size"], n_layer=hf["num_hidden_layers"], n_head=n_head,
        n_embd=hf["hidden_size"], n_query_groups=hf.get("num_key_value_heads", n_head), head_size=head_size,
        intermediate_size=hf["intermediate_size"], norm_eps=hf.get("rms_norm_eps", 1e-5),
        rope_base=int(_rope_theta(hf)), rotary_percentage=1.0, parallel_residual=False, bias=False,
        norm_class_name="RMSNorm", mlp_class_name="LLaMAMLP",
    )
    if "gemma2" in arch:
        n_layer = hf["num_hidden_layers"]
        layer_types = hf.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n_layer)]
        if "Gemma" not in kw["name"]:
            kw["name"] = "Gemma-2-" + kw["name"]  # the norm classes take their unit offset from the model name
        kw.update(
            mlp_class_name="GemmaMLP", gelu_approximate="tanh", scale_embeddings=True, post_attention_norm=True,
            post_mlp_norm=True, sliding_window_size=hf.get("sliding_window"),
            sliding_window_indices=[1 if t == "sliding_attention" else 0 for t in layer_types],
            attention_scores_scalar=hf.get("query_pre_attn_scalar"), attention_logit_softcapping=hf.get("attn_logit_softcapping"),
            final_logit_softcapping=hf.get("final_logit_softcapping"),
        )
    if "qwen2" in arch:
        kw["attn_bias"] = True
    if "qwen3" in arch:
        kw["norm_qk"] = True
    return Config(**kw)


def _iter_weight_files(hf_dir: Path) -> Iterable[Path]:
    files = sorted(hf_dir.glob("*.safetensors")) or sorted(hf_dir.glob("pytorch_model*.bin"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin in {hf_dir}")
    return files


def convert(hf_dir: Path, out_dir: Path, model_name: Optional[str] = None, dtype: Optional[torch.dtype] = None) -> Config:
    hf_dir, out_dir = Path(hf_dir), Path(out_dir)
    config = config_from_hf(json.loads((hf_dir / "config.json").read_text()), model_name)
    sd: Dict[str, torch.Tensor] = {}
    for f in _iter_weight_files(hf_dir):
        if f.suffix == ".safetensors":
            from safetensors.torch import load_file

            sd.update(load_file(str(f)))
        else:
            sd.update(torch.load(str(f), map_location="cpu", weights_only=True))
    out = convert_state_dict(sd, config)
    if dtype is not None:
        out = {k: v.to(dtype) for k, v in out.items()}
    out_dir.mkdir(parents=True, exist_ok=True)
    torch.save(out, out_dir / "lit_model.pth")
    config.save(out_dir)
    for extra in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "generation_config.json"):
        if (hf_dir / extra).exists():
            (out_dir / extra).write_bytes((hf_dir / extra).read_bytes())
    return config


def setup(hf_dir: Path, out_dir: Path, model_name: Optional[str] = None, dtype: Optional[str] = None) -> None:
    """Entry point of ``python -m keys_values_b200 convert_hf_checkpoint <hf_dir> <out_dir>``."""
    cfg = convert(Path(hf_dir), Path(out_dir), model_name, getattr(torch, dtype) if dtype else None)
    print(f"wrote {Path(out_dir) / 'lit_model.pth'} ({cfg.name}: {cfg.n_layer} layers, {cfg.n_embd} wide)")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("hf_dir", type=Path)
    ap.add_argument("out_dir", type=Path)
    ap.add_argument("--model-name", default=None, help="name in the model registry (default: derive the config from config.json)")
    ap.add_argument("--dtype", default=None, choices=[None, "bfloat16", "float16", "float32"])
    args = ap.parse_args()
    cfg = convert(args.hf_dir, args.out_dir, args.model_name, getattr(torch, args.dtype) if args.dtype else None)
    print(f"wrote {args.out_dir / 'lit_model.pth'} ({cfg.name}: {cfg.n_layer} layers, {cfg.n_embd} wide)")


if __name__ == "__main__":
    main()
