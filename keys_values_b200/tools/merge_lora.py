"""LoRA checkpoints: merge into the base weights, and import adapters trained with Hugging Face PEFT.

    python -m keys_values_b200.tools.merge_lora merge <finetune_out_dir/final> <base_checkpoint_dir> [--out DIR]
    python -m keys_values_b200.tools.merge_lora from-peft <adapter_dir> <base_checkpoint_dir> --out DIR

``merge`` loads the base model with the LoRA configuration stored next to the adapter
(``hyperparameters.yaml``), loads ``lit_model.lora.pth``, folds ``(alpha / r) · B A`` into the frozen
weights and writes a plain ``lit_model.pth`` that every command can load without LoRA.

``from-peft`` reads ``adapter_config.json`` + ``adapter_model.safetensors|bin`` (per-projection
``q_proj / k_proj / v_proj / o_proj`` and MLP adapters of a Llama-like decoder) and writes
``lit_model.lora.pth`` in this framework's layout, where q, k and v share one fused projection: the A
matrices of the enabled parts are stacked, the B matrices concatenated along the output features.
Parity: ``keys_values/scripts/convert_lora_to_litgpt/merge_qwen3_lora.py`` and its workflow notes.
"""
from __future__ import annotations

import argparse
import json
import re
from pathlib import Path
from typing import Dict, Optional

import torch
import yaml


def merge(lora_dir: Path, base_dir: Path, out_dir: Optional[Path] = None) -> Path:
    from keys_values_b200.finetune.args import LoRAArgs
    from keys_values_b200.finetune.utils import LIT_MODEL_FNAME, copy_config_files, load_model_checkpoint
    from keys_values_b200.models import lora as lora_mod

    lora_dir, base_dir = Path(lora_dir), Path(base_dir)
    out_dir = Path(out_dir) if out_dir is not None else lora_dir / "merged"
    hp = {}
    for d in (lora_dir, lora_dir.parent):
        if (d / "hyperparameters.yaml").is_file():
            hp = yaml.safe_load((d / "hyperparameters.yaml").read_text()) or {}
            break
    args = LoRAArgs(**hp["lora"]) if isinstance(hp.get("lora"), dict) else LoRAArgs()
    config = lora_mod.Config.from_checkpoint(base_dir, **args.config_kwargs())
    model = lora_mod.GPT(config)
    load_model_checkpoint(model, base_dir, lora_dir)
    lora_mod.merge_lora_weights(model)
    sd = {k.replace(".linear.", "."): v for k, v in model.state_dict().items() if "lora_" not in k}
    out_dir.mkdir(parents=True, exist_ok=True)
    torch.save({"model": sd}, out_dir / LIT_MODEL_FNAME)
    copy_config_files(base_dir, out_dir)
    return out_dir


_PEFT_KEY = re.compile(r".*layers\.(\d+)\.(self_attn|mlp)\.(\w+)\.lora_([AB])(?:\.\w+)?\.weight$")
_MLP_NAMES = {"gate_proj": "fc_1", "up_proj": "fc_2", "down_proj": "proj"}


def peft_to_lora_state_dict(peft_sd: Dict[str, torch.Tensor], enabled_qkv=("q_proj", "v_proj")) -> Dict[str, torch.Tensor]:
    """PEFT adapter tensors → ``transformer.h.N.attn.qkv.lora_A/B``, ``attn.proj.lora_A/B``, ``mlp.*``.
    ``enabled_qkv``: which of q/k/v carry an adapter (the fused layer stacks exactly these, in q, k, v order)."""
    per_layer: Dict[int, Dict[str, Dict[str, torch.Tensor]]] = {}
    for key, t in peft_sd.items():
        m = _PEFT_KEY.match(key)
        if m:
            per_layer.setdefault(int(m.group(1)), {}).setdefault(m.group(3), {})[m.group(4)] = t
    out: Dict[str, torch.Tensor] = {}
    for layer, mods in sorted(per_layer.items()):
        parts = [p for p in ("q_proj", "k_proj", "v_proj") if p in enabled_qkv]
        if any(p in mods for p in parts):
            missing = [p for p in parts if p not in mods]
            if missing:
                raise ValueError(f"layer {layer}: adapters for {missing} are missing (enabled_qkv = {enabled_qkv})")
            out[f"transformer.h.{layer}.attn.qkv.lora_A"] = torch.cat([mods[p]["A"] for p in parts], dim=0)
            out[f"transformer.h.{layer}.attn.qkv.lora_B"] = torch.cat([mods[p]["B"] for p in parts], dim=0)
        if "o_proj" in mods:
            out[f"transformer.h.{layer}.attn.proj.lora_A"] = mods["o_proj"]["A"]
            out[f"transformer.h.{layer}.attn.proj.lora_B"] = mods["o_proj"]["B"]
        for hf, ours in _MLP_NAMES.items():
            if hf in mods:
                out[f"transformer.h.{layer}.mlp.{ours}.lora_A"] = mods[hf]["A"]
                out[f"transformer.h.{layer}.mlp.{ours}.lora_B"] = mods[hf]["B"]
    return out


def from_peft(adapter_dir: Path, base_dir: Path, out_dir: Path) -> Path:
    from keys_values_b200.finetune.utils import LORA_WEIGHTS_FNAME

    adapter_dir, out_dir = Path(adapter_dir), Path(out_dir)
    cfg = json.loads((adapter_dir / "adapter_config.json").read_text())
    if (adapter_dir / "adapter_model.safetensors").is_file():
        from safetensors.torch import load_file

        peft_sd = load_file(str(adapter_dir / "adapter_model.safetensors"))
    else:
        peft_sd = torch.load(str(adapter_dir / "adapter_model.bin"), map_location="cpu", weights_only=True)
    targets = set(cfg.get("target_modules") or [])
    enabled = tuple(p for p in ("q_proj", "k_proj", "v_proj") if p in targets)
    sd = peft_to_lora_state_dict(peft_sd, enabled)
    out_dir.mkdir(parents=True, exist_ok=True)
    torch.save({"model": sd}, out_dir / LORA_WEIGHTS_FNAME)
    lora = dict(r=cfg.get("r", 8), alpha=cfg.get("lora_alpha", 16), dropout=cfg.get("lora_dropout", 0.0), query="q_proj" in targets,
                key="k_proj" in targets, value="v_proj" in targets, projection="o_proj" in targets,
                mlp=any(t in targets for t in _MLP_NAMES), head=False)
    (out_dir / "hyperparameters.yaml").write_text(yaml.safe_dump({"lora": lora, "checkpoint_dir": str(base_dir)}))
    return out_dir


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("command", choices=["merge", "from-peft"])
    ap.add_argument("adapter_dir", type=Path)
    ap.add_argument("base_dir", type=Path)
    ap.add_argument("--out", type=Path, default=None)
    a = ap.parse_args(argv)
    if a.command == "merge":
        print(merge(a.adapter_dir, a.base_dir, a.out))
    else:
        if a.out is None:
            ap.error("from-peft needs --out")
        print(from_peft(a.adapter_dir, a.base_dir, a.out))


if __name__ == "__main__":
    main()
