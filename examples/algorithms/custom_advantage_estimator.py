"""Registering a custom advantage estimator and training with it:

    python -m skyrl_b200.launch --nproc-per-node 8 examples/algorithms/custom_advantage_estimator.py \
        trainer.policy.model.path=qwen2.5-1.5b trainer.algorithm.advantage_estimator=centered_reward ...
"""

import sys

import torch

from skyrl_b200.algorithms.rl import register_advantage_estimator
from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp


@register_advantage_estimator("centered_reward")
def centered_reward(token_level_rewards, response_mask, index, **kwargs):
    """Sequence reward minus the batch mean, broadcast over the response tokens (no per-group statistics)."""
    scores = token_level_rewards.sum(-1)
    adv = (scores - scores.mean()).unsqueeze(-1) * response_mask
    return adv, adv


if __name__ == "__main__":
    BasePPOExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
