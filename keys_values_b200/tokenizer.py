"""Tokenizer wrapper over a checkpoint directory (role of ``litgpt.tokenizer.Tokenizer``):
``tokenizer.json`` (HF tokenizers) or ``tokenizer.model`` (SentencePiece), with BOS/EOS
handling from ``tokenizer_config.json`` / ``generation_config.json``."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, List, Optional, Union

import torch


class Tokenizer:
    def __init__(self, checkpoint_dir: Union[Path, str]) -> None:
        checkpoint_dir = Path(checkpoint_dir)
        if not checkpoint_dir.exists():
            raise NotADirectoryError(f"The checkpoint directory does not exist: {str(checkpoint_dir)}")
        self.model_name = checkpoint_dir.stem
        self.use_bos = self.check_if_bos_token_used(checkpoint_dir)
        self.bos_id: Optional[int] = None
        self.eos_id: Optional[int] = None
        if (vocabulary_path := checkpoint_dir / "tokenizer.json").is_file():
            from tokenizers import Tokenizer as HFTokenizer

            self.processor = HFTokenizer.from_file(str(vocabulary_path))
            self.backend = "huggingface"
            if (cfg_path := checkpoint_dir / "tokenizer_config.json").is_file():
                config = json.loads(cfg_path.read_text(encoding="utf-8"))
                for name in ("bos_token", "eos_token"):
                    tok = config.get(name)
                    if isinstance(tok, dict):
                        tok = tok.get("content")
                    if tok is not None:
                        setattr(self, name[:3] + "_id", self.token_to_id(tok))
            if (gen_path := checkpoint_dir / "generation_config.json").is_file():
                config = json.loads(gen_path.read_text(encoding="utf-8"))
                if self.bos_id is None:
                    self.bos_id = config.get("bos_token_id")
                if self.eos_id is None:
                    eos = config.get("eos_token_id")
                    self.eos_id = eos[0] if isinstance(eos, list) else eos
        elif (vocabulary_path := checkpoint_dir / "tokenizer.model").is_file():
            from sentencepiece import SentencePieceProcessor

            self.processor = SentencePieceProcessor(model_file=str(vocabulary_path))
            self.backend = "sentencepiece"
            self.bos_id, self.eos_id = self.processor.bos_id(), self.processor.eos_id()
        else:
            raise NotImplementedError(f"no tokenizer.json or tokenizer.model in {checkpoint_dir}")

    @property
    def vocab_size(self) -> int:
        if self.backend == "huggingface":
            return self.processor.get_vocab_size(with_added_tokens=False)
        return self.processor.vocab_size()

    def token_to_id(self, token: str) -> int:
        id_ = self.processor.token_to_id(token) if self.backend == "huggingface" else self.processor.piece_to_id(token)
        if id_ is None:
            raise ValueError(f"token {token!r} not found in the collection.")
        return id_

    @staticmethod
    def check_if_bos_token_used(checkpoint_dir: Path) -> bool:
        if not (p := checkpoint_dir / "tokenizer_config.json").is_file():
            return False
        config = json.loads(p.read_text(encoding="utf-8"))
        if "add_bos_token" in config:
            return bool(config["add_bos_token"])
        return config.get("tokenizer_class") == "LlamaTokenizer"

    def encode(self, string: str, device=None, bos: Optional[bool] = None, eos: bool = False, max_length: int = -1) -> torch.Tensor:
        tokens = self.processor.encode(string).ids if self.backend == "huggingface" else self.processor.encode(string)
        tokens = list(tokens)
        if bos or (bos is None and self.use_bos):
            if self.bos_id is None:
                raise NotImplementedError("This tokenizer does not have a defined bos token.")
            if not tokens or tokens[0] != self.bos_id:
                tokens = [self.bos_id] + tokens
        if eos and (not tokens or tokens[-1] != self.eos_id):
            tokens = tokens + [self.eos_id]
        if max_length > 0:
            tokens = tokens[:max_length]
        return torch.tensor(tokens, dtype=torch.int, device=device)

    def decode(self, tensor: Union[torch.Tensor, Iterable[int]]) -> str:
        tokens = [tensor.item()] if isinstance(tensor, torch.Tensor) and tensor.ndim == 0 else [int(t) for t in tensor]
        return self.processor.decode(tokens)

    def decode_stream(self, token_stream: Iterable[torch.Tensor]) -> Iterable[str]:
        ids: List[int] = []
        prev = ""
        for tok in token_stream:
            ids.append(int(tok))
            text = self.decode(ids)
            yield text[len(prev):]
            prev = text
