"""Stand-in for ``litgpt.tokenizer``: a wrapper over a ``tokenizer.json`` file."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Union

import torch


class Tokenizer:
    def __init__(self, checkpoint_dir: Union[Path, str]) -> None:
        from tokenizers import Tokenizer as HFTokenizer

        checkpoint_dir = Path(checkpoint_dir)
        if not (checkpoint_dir / "tokenizer.json").is_file():
            raise NotImplementedError(f"no tokenizer.json under {checkpoint_dir}")
        self.processor = HFTokenizer.from_file(str(checkpoint_dir / "tokenizer.json"))
        self.backend = "huggingface"
        self.model_name = checkpoint_dir.stem
        self.use_bos = False
        self.bos_id: Optional[int] = None
        self.eos_id: Optional[int] = None
        cfg = checkpoint_dir / "tokenizer_config.json"
        if cfg.is_file():
            config = json.loads(cfg.read_text(encoding="utf-8"))
            for key, attr in (("bos_token", "bos_id"), ("eos_token", "eos_id")):
                tok = config.get(key)
                if isinstance(tok, dict):
                    tok = tok.get("content")
                if tok is not None:
                    setattr(self, attr, self.processor.token_to_id(tok))
            self.use_bos = bool(config.get("add_bos_token", False))

    @property
    def vocab_size(self) -> int:
        return self.processor.get_vocab_size(with_added_tokens=False)

    def token_to_id(self, token: str) -> int:
        return self.processor.token_to_id(token)

    def encode(self, string: str, device=None, bos: Optional[bool] = None, eos: bool = False, max_length: int = -1) -> torch.Tensor:
        tokens = self.processor.encode(string).ids
        if (bos or (bos is None and self.use_bos)) and self.bos_id is not None and (not tokens or tokens[0] != self.bos_id):
            tokens = [self.bos_id] + tokens
        if eos and self.eos_id is not None and (not tokens or tokens[-1] != self.eos_id):
            tokens = tokens + [self.eos_id]
        if max_length > 0:
            tokens = tokens[:max_length]
        return torch.tensor(tokens, dtype=torch.int, device=device)

    def decode(self, tensor: torch.Tensor) -> str:
        tokens = [tensor.item()] if tensor.ndim == 0 else tensor.tolist()
        return self.processor.decode(tokens)
