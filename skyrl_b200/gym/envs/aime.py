"""AIME-style math environment: reward 1 when the last ``\\boxed{}`` (or ``Answer:`` line) matches
(reference: skyrl-gym/skyrl_gym/envs/aime/env.py)."""

from __future__ import annotations

import re
from typing import Any, Dict

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput
from .math_utils import last_boxed, math_equal


class AIMEEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras and "ground_truth" in extras["reward_spec"], "reward_spec.ground_truth is required"
        self.ground_truth = str(extras["reward_spec"]["ground_truth"])

    def step(self, action: str) -> BaseTextEnvStepOutput:
        pred = last_boxed(action)
        if pred is None:
            m = re.findall(r"(?i)answer\s*:\s*([^\n]+)", action)
            pred = m[-1] if m else None
        ok = math_equal(pred, self.ground_truth)
        return BaseTextEnvStepOutput(observations=[], reward=1.0 if ok else 0.0, done=True,
                                     metadata={"acc": ok, "pred": pred})
