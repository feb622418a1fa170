"""Environment API: ``init`` / ``step`` / ``close`` in the Gymnasium spirit, specialised for LLM agents.

Interface parity with skyrl-gym (skyrl-gym/skyrl_gym/core.py:12-97): ``step(action)`` returns a dict with
``observations``, ``reward``, ``done`` and optional ``metadata`` / ``postprocessed_action``.
"""

from __future__ import annotations

from typing import Any, Dict, Generic, Optional, SupportsFloat, Tuple, TypedDict, TypeVar

ObsType = TypeVar("ObsType")
ActType = TypeVar("ActType")


class EnvStepOutput(TypedDict, total=False):
    observations: Any
    reward: SupportsFloat
    done: bool
    metadata: Optional[Dict[str, Any]]
    postprocessed_action: Optional[str]


class Env(Generic[ObsType, ActType]):
    """Base environment. Subclasses override ``init`` and ``step``; ``close`` is optional."""

    def init(self, *args, **kwargs) -> Tuple[ObsType, Dict[str, Any]]:
        raise NotImplementedError

    def step(self, action: ActType) -> EnvStepOutput:
        raise NotImplementedError

    def close(self) -> None:
        return None

    def get_metrics(self) -> Dict[str, Any]:
        """Per-episode metrics reported after the trajectory ends."""
        return {}

    @staticmethod
    def aggregate_metrics(metrics: list) -> Dict[str, Any]:
        """Combine per-episode metric dicts: numeric values are averaged, others dropped."""
        if not metrics:
            return {}
        keys = set().union(*[m.keys() for m in metrics])
        out = {}
        for k in keys:
            vals = [m[k] for m in metrics if isinstance(m.get(k), (int, float, bool))]
            if vals:
                out[k] = sum(float(v) for v in vals) / len(vals)
        return out

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> bool:
        self.close()
        return False

    def __str__(self) -> str:
        return f"Env({type(self).__name__})"
