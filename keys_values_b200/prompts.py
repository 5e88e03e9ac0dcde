"""Prompt styles (role of ``litgpt.prompts``): a style turns an instruction into the text fed
to the model and names the stop tokens of the reply."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Tuple, Type, Union


class PromptStyle:
    def apply(self, prompt: str, **kwargs: str) -> str:
        return prompt

    def stop_tokens(self, tokenizer) -> Tuple[List[int], ...]:
        return ([tokenizer.eos_id],)

    @classmethod
    def from_name(cls, name: str) -> "PromptStyle":
        return prompt_styles[name]()


class Default(PromptStyle):
    pass


class Alpaca(PromptStyle):
    def apply(self, prompt: str, **kwargs: str) -> str:
        if kwargs.get("input"):
            return (
                "Below is an instruction that describes a task, paired with an input that provides further context. "
                "Write a response that appropriately completes the request.\\n\\n"
                f"### Instruction:\\n{prompt}\\n\\n### Input:\\n{kwargs['input']}\\n\\n### Response:\\n"
            )
        return (
            "Below is an instruction that describes a task. Write a response that appropriately completes the request.\\n\\n"
            f"### Instruction:\\n{prompt}\\n\\n### Response:\\n"
        )


class ChatML(PromptStyle):
    """Qwen / ChatML style."""

    system = "You are a helpful assistant."

    def apply(self, prompt: str, **kwargs: str) -> str:
        system = kwargs.get("sys_prompt") or self.system
        return f"<|im_start|>system\\n{system}<|im_end|>\\n<|im_start|>user\\n{prompt}<|im_end|>\\n<|im_start|>assistant\\n"


class Llama3(PromptStyle):
    def apply(self, prompt: str, **kwargs: str) -> str:
        system = kwargs.get("sys_prompt") or "You are a helpful assistant."
        return (
            f"<|begin_of_text|><|start_header_id|>system<|end_header_id|>\\n\\n{system}<|eot_id|>"
            f"<|start_header_id|>user<|end_header_id|>\\n\\n{prompt}<|eot_id|><|start_header_id|>assistant<|end_header_id|>\\n\\n"
        )

    def stop_tokens(self, tokenizer):
        return ([tokenizer.eos_id], [tokenizer.token_to_id("<|eot_id|>")])


prompt_styles: Dict[str, Type[PromptStyle]] = {"default": Default, "alpaca": Alpaca, "chatml": ChatML, "qwen": ChatML, "llama3": Llama3}


def save_prompt_style(style: Union[str, PromptStyle], checkpoint_dir: Path) -> None:
    name = style if isinstance(style, str) else next(k for k, v in prompt_styles.items() if isinstance(style, v))
    (Path(checkpoint_dir) / "prompt_style.yaml").write_text(json.dumps({"style": name}))


def has_prompt_style(checkpoint_dir: Path) -> bool:
    return (Path(checkpoint_dir) / "prompt_style.yaml").is_file()


def load_prompt_style(checkpoint_dir: Path) -> PromptStyle:
    cfg = json.loads((Path(checkpoint_dir) / "prompt_style.yaml").read_text())
    return PromptStyle.from_name(cfg["style"])
