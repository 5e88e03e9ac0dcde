"""Stand-in for the ``litgpt`` package (only the symbols the reference library imports)."""
from litgpt.config import Config  # noqa: F401
from litgpt.prompts import PromptStyle  # noqa: F401
from litgpt.tokenizer import Tokenizer  # noqa: F401
from litgpt import model, lora, utils  # noqa: F401

__all__ = ["Config", "PromptStyle", "Tokenizer"]
