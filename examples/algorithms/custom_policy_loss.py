"""Registering a custom policy loss (here: plain REINFORCE with a ratio cap) and training with it:

    python -m skyrl_b200.launch --nproc-per-node 8 examples/algorithms/custom_policy_loss.py \
        trainer.policy.model.path=qwen2.5-1.5b trainer.algorithm.policy_loss_type=capped_reinforce ...
"""

import sys

import torch

from skyrl_b200.algorithms.rl import reduce_loss, register_policy_loss
from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp


@register_policy_loss("capped_reinforce")
def capped_reinforce(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    ratio = torch.exp(log_probs - old_log_probs).clamp(max=2.0)
    loss = -(ratio.detach() * advantages * log_probs)
    return reduce_loss(loss, loss_mask), {"clip_ratio": float((ratio >= 2.0).float().mean())}


if __name__ == "__main__":
    BasePPOExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
