"""AIME / DAPO-style math environment: the response must end with an ``Answer: ...`` line; the answer is normalised the
Minerva way (units and wrappers stripped, TeX shorthand expanded) and compared as a string with the normalised ground
truth.  Reward ``+1`` for a match and ``-1`` otherwise, as in the DAPO recipe.  Reference: skyrl-gym/skyrl_gym/envs/
aime/{env,utils}.py (same extraction window, answer pattern, normalisation rules and scores, so that numbers carry over).
"""

from __future__ import annotations

import re
from typing import Any, Dict, Optional, Tuple

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput

# only the tail of a response can hold the final answer (the longest MATH-500 answer has 159 characters)
_TAIL_CHARS = 300
_ANSWER_LINE = re.compile(r"(?i)answer\s*:\s*([^\n<]+)")  # stops at a newline or at the '<' of an end-of-turn token

# rewrites applied in order (articles, spacing, \mbox, "and" inside tuples)
_REWRITES: Tuple[Tuple[str, str], ...] = (
    ("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), ("\\ ", ""), (" ", ""), ("mbox", "text"),
    (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}"),
)
# unit words and decorations that do not change the value of an answer
_IGNORED: Tuple[str, ...] = (
    "square", "ways", "integers", "dollars", "mph", "inches", "hours", "km", "units", "\\ldots", "sue", "points", "feet",
    "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges", "students",
    "childrentickets", "multiples", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}",
    "\\text{}", "\\mathrm{th}", "^\\circ", "^{\\circ}", "\\;", ",\\!", "{,}", '"', "\\dots",
)
_UNWRAP = tuple(re.compile(r"(\\%s\{)(.*?)(\})" % name) for name in ("text", "textbf", "overline"))
_UNBOX = re.compile(r"(\\boxed\{)(.*)(\})")
_INLINE_MATH = re.compile(r"(.*?)(\$)(.*?)(\$)(.*)")
_FRAC_SHORT = re.compile(r"(frac)([^{])(.)")
_SQRT_SHORT = re.compile(r"(sqrt)([^{])")


def normalize_final_answer(answer: str) -> str:
    """Right-hand side of the last ``=``; rewrites and ignored words removed; ``$...$`` reduced to its content;
    ``\\text{} / \\textbf{} / \\overline{} / \\boxed{}`` unwrapped; ``\\fracab -> \\frac{a}{b}``, ``\\sqrta -> \\sqrt{a}``;
    thousands separators dropped from plain integers."""
    s = answer.split("=")[-1]
    for old, new in _REWRITES:
        s = s.replace(old, new)
    for word in _IGNORED:
        s = s.replace(word, "")
    s = _INLINE_MATH.sub(r"$\3$", s)
    for pat in _UNWRAP:
        s = pat.sub(r"\2", s)
    s = _UNBOX.sub(r"\2", s)
    s = _FRAC_SHORT.sub(r"frac{\2}{\3}", s)
    s = _SQRT_SHORT.sub(r"sqrt{\2}", s)
    s = s.replace("$", "")
    if s.replace(",", "").isdigit():
        s = s.replace(",", "")
    return s.strip()


def last_boxed_only_string(text: str) -> Optional[str]:
    """The last ``\\boxed{...}`` of ``text`` with balanced braces, wrapper included; None if there is none."""
    start = text.rfind("\\boxed{")
    if start < 0:
        return None
    depth = 0
    for i in range(start, len(text)):
        if text[i] == "{":
            depth += 1
        elif text[i] == "}":
            depth -= 1
            if depth == 0:
                return text[start : i + 1]
    return None


def compute_score(solution: str, ground_truth: str, strict_box_verify: bool = False) -> Dict[str, Any]:
    """``{"score": +1 | -1, "acc": bool, "pred": str | None}``.  Default: the last ``Answer:`` line of the response's
    tail against the ground truth, both normalised.  ``strict_box_verify``: the last ``\\boxed{}`` within the final
    100 characters must equal the ground truth verbatim."""
    tail = solution[-_TAIL_CHARS:]
    if strict_box_verify:
        boxed = last_boxed_only_string(tail[-100:])
        pred = boxed[len("\\boxed{") : -1] if boxed is not None else None
        ok = pred == ground_truth
    else:
        found = _ANSWER_LINE.findall(tail)
        pred = normalize_final_answer(found[-1] if found else "[INVALID]")
        ok = pred == normalize_final_answer(ground_truth)
    return {"score": 1.0 if ok else -1.0, "acc": ok, "pred": pred}


class AIMEEnv(BaseTextEnv):
    """Single-turn.  The ground truth comes from ``extras["reward_model"]["ground_truth"]`` (the DAPO / AIME data
    layout the reference reads) or, for datasets written for the other environments here, ``extras["reward_spec"]``."""

    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        spec = extras.get("reward_model") or extras.get("reward_spec")
        assert spec is not None and "ground_truth" in spec, "reward_model.ground_truth (or reward_spec.ground_truth) is required"
        self.ground_truth = str(spec["ground_truth"])

    def step(self, action: str) -> BaseTextEnvStepOutput:
        info = compute_score(action, self.ground_truth)
        return BaseTextEnvStepOutput(observations=[], reward=info["score"], done=True,
                                     metadata={"acc": info["acc"], "pred": info["pred"]})
