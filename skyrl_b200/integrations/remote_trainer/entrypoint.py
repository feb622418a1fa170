"""``python -m skyrl_b200.integrations.remote_trainer.entrypoint --service-url http://host:port <config overrides>``

GRPO with the RL loop in this process and the model behind a Tinker-compatible training service (reference:
integrations/arctic_rl/entrypoint.py, which does the same against the Arctic RL server).  Start the service with
``python -m skyrl_b200.tinker.api`` (see ``examples/tinker``).
"""

from __future__ import annotations

import sys

from ...config.config import SkyRLTrainConfig
from ...entrypoints.main_base import BasePPOExp
from .client import TrainingServiceClient
from .trainer import RemoteBackendTrainer


class RemoteBackendExp(BasePPOExp):
    def __init__(self, cfg: SkyRLTrainConfig, service_url: str):
        self.service_url = service_url
        super().__init__(cfg)

    def get_inference_client(self):
        return None  # sampling goes through the service too

    def get_generator(self, cfg, tokenizer, inference_engine_client):
        return None  # built by the trainer around the service's sampler

    def get_trainer(self, cfg, tracker, tokenizer, train_dataset, eval_dataset, inference_engine_client, generator):
        return RemoteBackendTrainer(cfg, TrainingServiceClient(self.service_url), tracker=tracker, tokenizer=tokenizer,
                                    train_dataset=train_dataset, eval_dataset=eval_dataset, env=self.env)


def main(argv=None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--service-url" not in argv or argv.index("--service-url") + 1 >= len(argv):
        raise SystemExit("give --service-url http://host:port of the training service")
    i = argv.index("--service-url")
    url = argv[i + 1]
    cfg = SkyRLTrainConfig.from_cli_overrides(argv[:i] + argv[i + 2:])
    RemoteBackendExp(cfg, url).run()


if __name__ == "__main__":
    main()
