"""Built-in tools for the agent runners and a registry to look them up by name.

Reference (peripheral package): skyrl-agent/skyrl_agent/tools (finish / em_finish, local_search, sandbox code
execution).  Every tool is a plain callable wrapped in ``react.Tool``; results are text the model reads next.
"""

from __future__ import annotations

import math
import re
import subprocess
import sys
import tempfile
from collections import Counter
from typing import Any, Callable, Dict, List, Optional, Sequence

from .react import Tool

TOOL_REGISTRY: Dict[str, Callable[..., Tool]] = {}


def register_tool(name: str):
    def deco(factory: Callable[..., Tool]):
        TOOL_REGISTRY[name] = factory
        return factory

    return deco


def make_tool(name: str, **kwargs) -> Tool:
    if name not in TOOL_REGISTRY:
        raise KeyError(f"unknown tool '{name}'; registered: {sorted(TOOL_REGISTRY)}")
    return TOOL_REGISTRY[name](**kwargs)


@register_tool("finish")
def finish_tool() -> Tool:
    """Ends the episode with an answer (agents that prefer a tool call over an ``<answer>`` block)."""
    return Tool("finish", lambda answer="": f"<answer>{answer}</answer>", "finish(answer): end the task with your final answer")


def normalize_answer(s: str) -> str:
    """Lower-case, strip punctuation, articles and extra white space (the usual exact-match normalisation)."""
    s = re.sub(r"[^\w\s]", " ", str(s).lower())
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def exact_match(prediction: Optional[str], golds: Sequence[str]) -> float:
    if prediction is None:
        return 0.0
    p = normalize_answer(prediction)
    return 1.0 if any(p == normalize_answer(g) for g in golds) else 0.0


@register_tool("python")
def python_tool(timeout: float = 5.0, max_output: int = 2000) -> Tool:
    """Runs a code snippet in a fresh interpreter (separate process, isolated mode, time limit, truncated output)."""

    def run(code: str = "") -> str:
        with tempfile.TemporaryDirectory() as d:
            try:
                p = subprocess.run([sys.executable, "-I", "-c", code], capture_output=True, text=True, timeout=timeout, cwd=d)
                out = p.stdout + (("\n[stderr]\n" + p.stderr) if p.stderr else "")
                if p.returncode != 0:
                    out += f"\n[exit code {p.returncode}]"
            except subprocess.TimeoutExpired:
                out = f"[timed out after {timeout} s]"
        return out[:max_output] if out else "[no output]"

    return Tool("python", run, "python(code): run Python code, returns what it printed")


class BM25Index:
    """A small in-memory BM25 index over text passages (stands in for the reference's retrieval server)."""

    def __init__(self, passages: Sequence[str], k1: float = 1.5, b: float = 0.75):
        self.passages = list(passages)
        self.docs = [self._tok(p) for p in self.passages]
        self.k1, self.b = k1, b
        self.avg = sum(len(d) for d in self.docs) / max(1, len(self.docs))
        self.df: Counter = Counter()
        for d in self.docs:
            self.df.update(set(d))

    @staticmethod
    def _tok(s: str) -> List[str]:
        return re.findall(r"\w+", s.lower())

    def search(self, query: str, top_k: int = 3) -> List[str]:
        q = self._tok(query)
        N = len(self.docs)
        scores = []
        for i, d in enumerate(self.docs):
            tf = Counter(d)
            s = 0.0
            for t in q:
                if t not in tf:
                    continue
                idf = math.log(1 + (N - self.df[t] + 0.5) / (self.df[t] + 0.5))
                s += idf * tf[t] * (self.k1 + 1) / (tf[t] + self.k1 * (1 - self.b + self.b * len(d) / max(1e-9, self.avg)))
            scores.append((s, i))
        best = sorted(scores, key=lambda x: (-x[0], x[1]))[:top_k]
        return [self.passages[i] for s, i in best if s > 0]


@register_tool("local_search")
def local_search_tool(passages: Sequence[str] = (), top_k: int = 3) -> Tool:
    index = BM25Index(passages)

    def search(query: str = "") -> str:
        hits = index.search(query, top_k)
        return "\n".join(f"[{i + 1}] {h}" for i, h in enumerate(hits)) if hits else "no results"

    return Tool("local_search", search, "local_search(query): look up passages in the local corpus")
