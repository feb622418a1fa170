"""Entry point for the REPL-driven long-context environment with recursive sub-calls: the trainer's generator is the
``RLMGenerator``, which lets the code the policy writes call ``llm_query`` / ``rlm_query`` (plain generations and child
episodes served by the same colocated engine)."""

import sys

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp
from skyrl_b200.train.generators.rlm_generator import RLMGenerator


class RLMExp(BasePPOExp):
    max_depth = 1

    def _setup_trainer(self):
        trainer = super()._setup_trainer()
        trainer.generator = RLMGenerator(self.cfg.generator, self.cfg.environment.skyrl_gym, trainer.inference_engine_client,
                                         self.tokenizer, max_depth=self.max_depth, subcall_max_tokens=512)
        return trainer


if __name__ == "__main__":
    RLMExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
