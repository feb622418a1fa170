"""Experiment class for the one-step-off-policy trainer; selected with
``trainer.override_entrypoint=examples.async.one_step_off:Exp`` (see run_one_step_off.sh)."""

from skyrl_b200.entrypoints.main_base import BasePPOExp
from skyrl_b200.train.async_trainer import OneStepOffPPOTrainer


class Exp(BasePPOExp):
    def get_trainer(self, cfg, tracker, tokenizer, train_dataset, eval_dataset, inference_engine_client, generator):
        return OneStepOffPPOTrainer(cfg, tracker=tracker, tokenizer=tokenizer, train_dataset=train_dataset,
                                    eval_dataset=eval_dataset, inference_engine_client=inference_engine_client,
                                    generator=generator, env=self.env)
