"""GSM8K environments: single-turn exact-match reward and a multi-turn variant that gives feedback.

Behavioural reference: skyrl-gym/skyrl_gym/envs/gsm8k/env.py and gsm8k_multi_turn/env.py.
``extras`` must carry ``reward_spec = {"method": "rule", "ground_truth": <str>}``.
"""

from __future__ import annotations

from typing import Any, Dict

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput
from .math_utils import extract_gsm8k_answer


class GSM8kEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        assert "reward_spec" in extras, "reward_spec field is required"
        assert "ground_truth" in extras["reward_spec"], "ground_truth is required in reward_spec field"
        self.ground_truth = str(extras["reward_spec"]["ground_truth"])

    def _score(self, action: str) -> float:
        ans = extract_gsm8k_answer(action, "strict")
        return 1.0 if ans is not None and ans == self.ground_truth else 0.0

    def step(self, action: str) -> BaseTextEnvStepOutput:
        return BaseTextEnvStepOutput(observations=[], reward=self._score(action), done=True, metadata={})


class GSM8kMultiTurnEnv(GSM8kEnv):
    """Up to ``max_turns`` attempts; a wrong or missing answer produces a user message asking to retry."""

    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__(env_config, extras)
        self.max_turns = int((extras or {}).get("max_turns", 5))

    def step(self, action: str) -> BaseTextEnvStepOutput:
        self.turns += 1
        found = extract_gsm8k_answer(action, "strict")
        correct = found is not None and found == self.ground_truth
        if correct:
            return BaseTextEnvStepOutput(observations=[], reward=1.0, done=True, metadata={"parsed": found})
        if self.turns >= self.max_turns:
            return BaseTextEnvStepOutput(observations=[], reward=0.0, done=True, metadata={"parsed": found})
        if found is None:
            msg = "Please give your final answer in the format '#### <number>'."
        else:
            msg = "Your previous answer is incorrect. Please re-check your reasoning and answer again."
        small = 0.2 / self.max_turns if found is not None else 0.0  # tiny format reward on intermediate turns
        return BaseTextEnvStepOutput(observations=[{"role": "user", "content": msg}], reward=small, done=False,
                                     metadata={"parsed": found})
