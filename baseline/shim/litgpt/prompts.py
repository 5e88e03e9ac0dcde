"""Stand-in for ``litgpt.prompts``."""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Tuple, Type, Union

import yaml


class PromptStyle:
    def apply(self, prompt: str, **kwargs: str) -> str:
        return prompt

    def stop_tokens(self, tokenizer) -> Tuple[List[int], ...]:
        return ([tokenizer.eos_id],)

    @classmethod
    def from_name(cls, name: str) -> "PromptStyle":
        return prompt_styles[name]()

    @classmethod
    def from_config(cls, config) -> "PromptStyle":
        return Default()


class Default(PromptStyle):
    pass


prompt_styles: Dict[str, Type[PromptStyle]] = {"default": Default}


def save_prompt_style(style: Union[str, PromptStyle], checkpoint_dir: Path) -> None:
    style = PromptStyle.from_name(style) if isinstance(style, str) else style
    name = {v: k for k, v in prompt_styles.items()}.get(type(style), "default")
    with open(Path(checkpoint_dir) / "prompt_style.yaml", "w", encoding="utf-8") as fp:
        yaml.dump({"style_name": name}, fp)


def load_prompt_style(checkpoint_dir: Path) -> PromptStyle:
    with open(Path(checkpoint_dir) / "prompt_style.yaml", encoding="utf-8") as fp:
        return PromptStyle.from_name(yaml.safe_load(fp)["style_name"])


def has_prompt_style(checkpoint_dir: Path) -> bool:
    return (Path(checkpoint_dir) / "prompt_style.yaml").is_file()
