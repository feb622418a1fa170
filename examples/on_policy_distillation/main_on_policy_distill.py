"""On-policy distillation: the student samples, a larger teacher scores the samples, and the per-token reward is the
negative reverse-KL estimate ``-(log pi_student - log pi_teacher)``; no task reward, no environment signal.

The teacher takes the place of the reference model (``trainer.ref.model.path``), ``use_kl_in_reward`` routes the
batch through ``apply_reward_kl_penalty``, and a pass-through advantage estimator hands the rewards to the loss.
"""

import sys

from skyrl_b200.algorithms.rl import register_advantage_estimator
from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp
from skyrl_b200.train.trainer import PPOTrainer


@register_advantage_estimator("token_rewards")
def token_rewards(token_level_rewards, response_mask, index=None, **kwargs):
    adv = token_level_rewards * response_mask
    return adv, adv


class DistillationTrainer(PPOTrainer):
    def apply_reward_kl_penalty(self, batch):
        mask = batch["loss_mask"]
        gap = (batch["action_log_probs"] - batch["base_action_log_probs"]) * mask
        batch["rewards"] = -gap
        self.all_metrics["distill/student_minus_teacher_logprob"] = float(gap.sum() / mask.sum().clamp(min=1))
        return batch


class DistillationExp(BasePPOExp):
    def get_trainer(self, cfg, tracker, tokenizer, train_dataset, eval_dataset, inference_engine_client, generator):
        return DistillationTrainer(cfg, tracker=tracker, tokenizer=tokenizer, train_dataset=train_dataset,
                                   eval_dataset=eval_dataset, inference_engine_client=inference_engine_client,
                                   generator=generator, env=self.env)


if __name__ == "__main__":
    DistillationExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
