"""A tiny custom environment: "what is A times B?" with a numeric answer, two attempts.

Shows the three pieces a new task needs: an environment class, its registration, and a dataset whose rows carry the
prompt and whatever the environment wants in ``extra_info`` / ``reward_spec``.
"""

import re
from typing import Any, Dict

from skyrl_b200.gym.envs.base_text_env import BaseTextEnv, BaseTextEnvStepOutput


class MultiplyEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        self.answer = str((extras.get("reward_spec") or {}).get("ground_truth", extras.get("ground_truth", "")))
        self.max_turns = int(extras.get("max_turns", 2))

    @staticmethod
    def _last_number(text: str):
        found = re.findall(r"-?\d+", text.replace(",", ""))
        return found[-1] if found else None

    def step(self, action: str) -> BaseTextEnvStepOutput:
        self.turns += 1
        guess = self._last_number(action)
        if guess is not None and guess == self.answer:
            return BaseTextEnvStepOutput(observations=[], reward=1.0, done=True, metadata={"turns": self.turns})
        if self.turns >= self.max_turns:
            # a well-formed but wrong answer is worth a little more than no number at all
            return BaseTextEnvStepOutput(observations=[], reward=0.1 if guess is not None else 0.0, done=True,
                                         metadata={"turns": self.turns})
        hint = "That is not right. Multiply digit by digit and answer with the number only."
        return BaseTextEnvStepOutput(observations=[{"role": "user", "content": hint}], reward=0.0, done=False, metadata={})
