"""GRPO with rollouts driven through the OpenAI-compatible endpoint (see ``chat_generator.py``)."""

import sys

from examples.train_integrations.openai_chat.chat_generator import ChatCompletionsGenerator
from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp


class ChatExp(BasePPOExp):
    def _setup_trainer(self):
        trainer = super()._setup_trainer()
        # the trainer built its colocated engine; put the chat-protocol generator in front of it
        trainer.generator = ChatCompletionsGenerator(self.cfg.generator, self.cfg.environment.skyrl_gym,
                                                     trainer.inference_engine_client, self.tokenizer)
        return trainer


if __name__ == "__main__":
    ChatExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
