"""Entry point that registers the environment before the trainer starts (one process per GPU runs this file)."""

import sys

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.entrypoints.main_base import BasePPOExp
from skyrl_b200.gym import register

register("multiply", "examples.multiply.env:MultiplyEnv", override=True)

if __name__ == "__main__":
    BasePPOExp(SkyRLTrainConfig.from_cli_overrides(sys.argv[1:])).run()
