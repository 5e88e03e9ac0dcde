"""Turning a generated reply into the thing a metric compares (``keys_values/evaluation/response_parser.py``).

Models wrap answers in lead-ins ("Answer:", "the label is …"), quotes, markdown and trailing chatter. These
helpers pull out the normalised string, the numbers, the multiple-choice letter or the value token."""
from __future__ import annotations

import re
from typing import List, Optional, Sequence, Union

_LEAD_WORDS = ("answer", "document", "response", "output", "label", "</think>")
_FIELD_WORDS = ("answer", "label", "document", "response", "output")


def parse_answer(text: str, prefix: str = "Answer:") -> str:
    """Text after the last ``prefix`` up to the end of that line; the whole first line if absent."""
    idx = text.rfind(prefix)
    body = (text[idx + len(prefix):] if idx >= 0 else text).strip()
    return body.split("\n")[0].strip() if body else ""


def normalize_string_response(text: Optional[str], *, prefixes: Sequence[str] = _LEAD_WORDS) -> str:
    """Strips white space, any stack of leading prefixes ("Answer:", "Label -", "</think>" …, case-insensitive),
    a lead-in clause within the first 240 characters that ends in "… the answer is:" / "label =" and the like, and
    one layer of surrounding quotes or back-ticks."""
    if text is None:
        return ""
    s = str(text).strip()
    if not s:
        return ""
    words = [re.escape(p) for p in prefixes if p]
    if words:
        lead = re.compile(r"^(?:" + "|".join(words) + r")\s*(?:[:=\-]\s*|\s+)?", re.IGNORECASE)
        while True:
            shorter = lead.sub("", s, count=1).lstrip()
            if shorter == s:
                break
            s = shorter
    clause = re.compile(r"(?is)^.*?\b(?:the\s+)?(?:" + "|".join(_FIELD_WORDS) + r")\b\s*(?:is\b\s*)?(?:[:=\-]\s*|\s+)")
    hit = clause.search(s[:240])
    if hit:
        s = s[hit.end():].lstrip()
    if len(s) >= 2 and s[0] == s[-1] and s[0] in "`\"'":
        s = s[1:-1].strip()
    return s


_NUMBER = re.compile(r"(?<![\w.])[-+]?(?:\d{1,3}(?:,\d{3})+|\d+)(?:\.\d+)?(?:[eE][-+]?\d+)?(?:\.(?=\s*(?!\d)))?(?![\w.])")


def extract_numbers(text: str, *, as_list: bool = True) -> Union[List[str], str]:
    """Numbers in free text (thousands separators, decimals, exponents), each as the string of its integer part;
    ``["0"]`` (or ``"0"``) when there is none. With ``as_list=False`` the first one."""
    found: List[str] = []
    for m in _NUMBER.findall(text or ""):
        try:
            found.append(str(int(float(m.replace(",", "").rstrip(".")))))
        except ValueError:
            continue
    if as_list:
        return found or ["0"]
    return found[0] if found else "0"


def parse_ranked_ids(text: str) -> List[str]:
    return re.findall(r"\d+", text)


_LETTER = re.compile(r"(?<![A-Za-z0-9])[\(\[\{'\"]*(?P<ch>[A-Za-z])[\)\]\}'\"]*[\.\):,\-]?(?![A-Za-z0-9])")
_CHOICE_CUE = re.compile(r"\b(answer|correct|option|choice|select|selected|pick)\b", re.IGNORECASE)


def extract_choice_letter(text: str, *, choices: str = "ABCD", default: str = "") -> str:
    """The multiple-choice letter of a reply: stand-alone letters in any of the forms ``C``, ``C.``, ``(C)``,
    ``option D``; a letter within 40 characters of a cue word (answer, correct, option, choice, select, pick) wins
    over one without, later ones over earlier ones."""
    allowed = {c.upper() for c in choices if c.strip()}
    if not text or not allowed:
        return default
    best = None
    for m in _LETTER.finditer(text):
        ch = m.group("ch").upper()
        if ch not in allowed:
            continue
        near_cue = bool(_CHOICE_CUE.search(text[max(0, m.start() - 40): m.end() + 40]))
        key = (near_cue, m.start())
        if best is None or key >= best[0]:
            best = (key, ch)
    return best[1] if best else default


_HEXISH = re.compile(r"\b[0-9a-fA-F]{4,}(?:-[0-9a-fA-F]{1,})+\b")
_INT = re.compile(r"\b\d+\b")


def _value_in(chunk: str) -> Optional[str]:
    quoted = re.search(r"`([^`]+)`", chunk)
    for part in ([quoted.group(1).strip()] if quoted else []) + [chunk]:
        for pattern in (_HEXISH, _INT):
            m = pattern.search(part)
            if m:
                return m.group(0)
    return None


def extract_value_token(text: str, *, default: str = "") -> str:
    """The value a recall task asks for (a UUID-like hyphenated hex token or an integer): the first one after a cue
    "is" / "are" (optionally with a colon, markdown bold or back-ticks in between), else the last such token."""
    if not text:
        return default
    for cue in re.finditer(r"\b(?:is|are)\b\s*:?\s*", text, re.IGNORECASE):
        tail = text[cue.end(): cue.end() + 240].lstrip(" \t\r\n:=-")
        tail = re.sub(r"^(?:\*\*|__)+", "", tail).lstrip()
        val = _value_in(tail)
        if val:
            return val
    for pattern in (_HEXISH, _INT):
        all_found = pattern.findall(text)
        if all_found:
            return all_found[-1]
    return default
