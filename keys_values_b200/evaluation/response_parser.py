"""Extraction of the answer part of a generated reply (``keys_values/evaluation/response_parser.py``)."""
from __future__ import annotations

import re
from typing import List


def parse_answer(text: str, prefix: str = "Answer:") -> str:
    """Text after the last ``prefix`` up to the end of that line; the whole first line if absent."""
    idx = text.rfind(prefix)
    body = text[idx + len(prefix):] if idx >= 0 else text
    body = body.strip()
    return body.split("\n")[0].strip() if body else ""


def parse_ranked_ids(text: str) -> List[str]:
    return re.findall(r"\d+", text)
