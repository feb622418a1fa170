"""LLM-as-a-judge environment: the reward of a response is what a judge model says about it.

The judge is any OpenAI-compatible ``/v1/chat/completions`` endpoint -- a hosted model, or this package's own
inference server (``python -m skyrl_b200.entrypoints.serve``).  Behavioural reference: the reference's example
environment (examples/train/llm_as_a_judge/llm_judge_env.py), which asks a hosted judge to compare the answer with
the gold solution and rewards 1 / 0.

``extras``: ``reward_spec.ground_truth`` (gold answer shown to the judge) and optionally ``question``.
``env_config`` (``environment.skyrl_gym.llm_judge.*`` or a plain dict): ``base_url``, ``model``, ``api_key_env``
(name of the environment variable that holds the key), ``timeout``, ``max_retries``, ``prompt`` (template with
``{question}``, ``{gold}``, ``{answer}``).
"""

from __future__ import annotations

import json
import os
import re
import time
import urllib.error
import urllib.request
from typing import Any, Dict

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput

DEFAULT_PROMPT = (
    "You are grading an answer.\nQuestion: {question}\nGold answer: {gold}\nCandidate answer: {answer}\n"
    "Reply with a single line 'SCORE: x' where x is 1 if the candidate's final answer matches the gold answer and 0 "
    "otherwise.")


def _cfg(env_config: Any, key: str, default: Any) -> Any:
    if env_config is None:
        return default
    if isinstance(env_config, dict):
        return env_config.get(key, default)
    return getattr(env_config, key, default)


def parse_score(text: str) -> float | None:
    """``SCORE: x`` (last occurrence wins), clamped to [0, 1]; None when the judge did not follow the format."""
    found = re.findall(r"SCORE:\s*(-?\d+(?:\.\d+)?)", text or "", flags=re.IGNORECASE)
    if not found:
        return None
    return max(0.0, min(1.0, float(found[-1])))


class LLMJudgeEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        self.gold = str((extras.get("reward_spec") or {}).get("ground_truth", ""))
        self.question = str(extras.get("question", ""))
        self.base_url = str(_cfg(env_config, "base_url", os.environ.get("SKYRL_B200_JUDGE_URL", "http://127.0.0.1:8000"))).rstrip("/")
        self.model = str(_cfg(env_config, "model", "judge"))
        self.key = os.environ.get(str(_cfg(env_config, "api_key_env", "OPENAI_API_KEY")), "")
        self.timeout = float(_cfg(env_config, "timeout", 60.0))
        self.max_retries = int(_cfg(env_config, "max_retries", 3))
        self.prompt = str(_cfg(env_config, "prompt", DEFAULT_PROMPT))

    def _ask(self, content: str) -> str:
        body = json.dumps({"model": self.model, "messages": [{"role": "user", "content": content}], "temperature": 0.0,
                           "max_tokens": 64}).encode()
        headers = {"Content-Type": "application/json"}
        if self.key:
            headers["Authorization"] = f"Bearer {self.key}"
        last: Exception | None = None
        for attempt in range(self.max_retries):
            try:
                req = urllib.request.Request(self.base_url + "/v1/chat/completions", data=body, headers=headers)
                with urllib.request.urlopen(req, timeout=self.timeout) as r:
                    return json.loads(r.read())["choices"][0]["message"]["content"]
            except (urllib.error.URLError, TimeoutError, KeyError, json.JSONDecodeError) as e:
                last = e
                time.sleep(min(2.0, 0.2 * (attempt + 1)))
        raise RuntimeError(f"judge at {self.base_url} did not answer after {self.max_retries} attempts: {last}")

    def step(self, action: str) -> BaseTextEnvStepOutput:
        verdict = self._ask(self.prompt.format(question=self.question, gold=self.gold, answer=action))
        score = parse_score(verdict)
        return BaseTextEnvStepOutput(observations=[], reward=0.0 if score is None else score, done=True,
                                     metadata={"judge_reply": verdict, "judge_parsed": score is not None})
