"""Stand-in for ``litgpt.parser_config``."""
from pathlib import Path
from typing import Callable, List, Optional


def parser_commands() -> List[str]:
    return ["download", "chat", "finetune", "finetune_lora", "finetune_full", "pretrain", "generate", "evaluate"]


def save_hyperparameters(function: Callable, checkpoint_dir: Path, known_commands: Optional[List[str]] = None) -> None:
    raise NotImplementedError("litgpt.parser_config.save_hyperparameters is not provided by the stand-in package")
