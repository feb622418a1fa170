"""Answer extraction and comparison helpers for math-style rewards."""

from __future__ import annotations

import re
from typing import Optional


def extract_gsm8k_answer(text: str, method: str = "strict") -> Optional[str]:
    """``#### 42`` format (strict) or the last number in the text (flexible)."""
    if method == "strict":
        m = re.findall(r"#### (\-?[0-9\.\,]+)", text)
        if not m:
            return None
        return m[-1].replace(",", "").replace("$", "")
    nums = re.findall(r"(\-?[0-9\.\,]+)", text)
    for cand in reversed(nums):
        if cand not in ("", "."):
            return cand.replace(",", "")
    return None


def last_boxed(text: str) -> Optional[str]:
    """Content of the last ``\\boxed{...}`` with balanced braces."""
    idx = text.rfind("\\boxed")
    if idx < 0:
        return None
    i = text.find("{", idx)
    if i < 0:
        return None
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1 : j]
    return None


def normalize_math(s: str) -> str:
    s = s.strip().replace(" ", "").replace("\\!", "").replace("$", "").replace("\\%", "").replace("%", "")
    s = s.replace("dfrac", "frac").replace("tfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = re.sub(r"\\text\{(.*?)\}", r"\1", s)
    s = s.rstrip(".")
    if re.fullmatch(r"-?\d+\.0+", s):
        s = s.split(".")[0]
    return s


def math_equal(pred: Optional[str], truth: str) -> bool:
    if pred is None:
        return False
    a, b = normalize_math(pred), normalize_math(str(truth))
    if a == b:
        return True
    try:
        return abs(float(a) - float(b)) < 1e-6
    except ValueError:
        return False
