"""Tasks: what an agent is asked and how its result is scored.

Reference (peripheral package): skyrl-agent/skyrl_agent/tasks (``BaseTask`` with instruction / runtime
initialisation / evaluation hooks; general ReAct question answering, SWE-bench, web research).  A task here has three
asynchronous stages so that the pipeline dispatcher can overlap them across trajectories: ``initialize`` (set up
whatever the episode needs), the agent run itself, and ``evaluate`` (score the result).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from .react import AgentResult
from .tools import exact_match

TASK_REGISTRY: Dict[str, type] = {}


def register_task(name: str):
    def deco(cls):
        TASK_REGISTRY[name] = cls
        return cls

    return deco


class BaseTask:
    """One instance of a task.  ``instance`` is the dataset row."""

    def __init__(self, instance: Dict[str, Any]):
        self.instance = instance

    def instruction(self) -> str:
        raise NotImplementedError

    async def initialize(self) -> None:
        """Per-episode set-up (start a sandbox, fetch a repository, ...).  Nothing by default."""

    async def evaluate(self, result: AgentResult) -> float:
        raise NotImplementedError

    async def close(self) -> None:
        """Release what ``initialize`` acquired."""


@register_task("general_react")
class GeneralReactTask(BaseTask):
    """Question answering with exact-match scoring: rows carry ``question`` (or ``prompt``) and ``answer`` /
    ``golden_answers`` / ``reward_spec.ground_truth``."""

    def instruction(self) -> str:
        return str(self.instance.get("question", self.instance.get("prompt", "")))

    def golds(self) -> List[str]:
        row = self.instance
        g: Optional[Any] = row.get("golden_answers") or row.get("answer") or (row.get("reward_spec") or {}).get("ground_truth")
        if g is None:
            return []
        return [str(x) for x in g] if isinstance(g, (list, tuple)) else [str(g)]

    async def evaluate(self, result: AgentResult) -> float:
        return exact_match(result.answer, self.golds())
