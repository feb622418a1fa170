"""Synthetic environments for plumbing runs and benchmarks (no dataset, no external service).

* ``synthetic_bernoulli``  - single turn, reward ~ Bernoulli(p) (seeded per trajectory).
* ``synthetic_gaussian``   - single turn, reward ~ N(mean, std) (seeded per trajectory).
* ``synthetic_even``       - single turn, reward = fraction of response token ids that are even
                              (the response text is the space-separated ids of ``SyntheticTokenizer``).
* ``synthetic_multiturn``  - ``max_turns`` turns; every non-final turn returns an observation of
                              ``obs_tokens`` random token ids; reward ~ Bernoulli(p) at episode end.
"""

from __future__ import annotations

import random
from typing import Any, Dict

from .base_text_env import BaseTextEnv, BaseTextEnvStepOutput


class SyntheticBernoulliEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        self.p = float(extras.get("p", 0.5))
        seed = extras.get("seed", None)
        if seed is not None:  # distinct draws for the repetitions of one prompt
            seed = int(seed) * 1000003 + int(extras.get("repetition_id", 0))
        self.rng = random.Random(seed)

    def step(self, action: str) -> BaseTextEnvStepOutput:
        return BaseTextEnvStepOutput(observations=[], reward=1.0 if self.rng.random() < self.p else 0.0, done=True,
                                     metadata={})


class SyntheticGaussianEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        self.mean, self.std = float(extras.get("mean", 0.0)), float(extras.get("std", 1.0))
        seed = extras.get("seed", None)
        if seed is not None:
            seed = int(seed) * 1000003 + int(extras.get("repetition_id", 0))
        self.rng = random.Random(seed)

    def step(self, action: str) -> BaseTextEnvStepOutput:
        return BaseTextEnvStepOutput(observations=[], reward=self.rng.gauss(self.mean, self.std), done=True, metadata={})


class SyntheticEvenEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()

    def step(self, action: str) -> BaseTextEnvStepOutput:
        ids = [int(t) for t in action.split() if t.lstrip("-").isdigit()]
        frac = sum(1 for t in ids if t % 2 == 0) / max(1, len(ids))
        return BaseTextEnvStepOutput(observations=[], reward=frac, done=True, metadata={"n_tokens": len(ids)})


class SyntheticMultiTurnEnv(BaseTextEnv):
    def __init__(self, env_config: Any = None, extras: Dict[str, Any] | None = None):
        super().__init__()
        extras = extras or {}
        self.max_turns = int(extras.get("max_turns", 8))
        self.obs_tokens = int(extras.get("obs_tokens", 512))
        self.vocab = int(extras.get("vocab_size", 1024))
        self.p = float(extras.get("p", 0.3))
        self.rng = random.Random(extras.get("seed", None))

    def step(self, action: str) -> BaseTextEnvStepOutput:
        self.turns += 1
        if self.turns >= self.max_turns:
            return BaseTextEnvStepOutput(observations=[], reward=1.0 if self.rng.random() < self.p else 0.0, done=True,
                                         metadata={"turns": self.turns})
        obs = " ".join(str(self.rng.randrange(4, self.vocab)) for _ in range(self.obs_tokens))
        return BaseTextEnvStepOutput(observations=[{"role": "user", "content": obs}], reward=0.0, done=False, metadata={})
