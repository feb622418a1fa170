"""SFT entry point (reference: skyrl/train/entrypoints/main_sft.py:27-76).

    python -m skyrl_b200.entrypoints.main_sft model.path=... dataset_name=train.jsonl batch_size=64
    python -m skyrl_b200.launch --nproc-per-node 8 -m skyrl_b200.entrypoints.main_sft ...
"""

from __future__ import annotations

import sys
from typing import List, Optional

from ..config.sft_config import SFTConfig
from ..parallel import dist as pdist
from ..train.sft_trainer import SFTTrainer


def sft_entrypoint(cfg: SFTConfig) -> dict:
    env = pdist.init_distributed()
    try:
        trainer = SFTTrainer(cfg, env=env).setup()
        return trainer.train()
    finally:
        pdist.shutdown()


def main(argv: Optional[List[str]] = None) -> None:
    sft_entrypoint(SFTConfig.from_cli_overrides(sys.argv[1:] if argv is None else argv))


if __name__ == "__main__":
    main()
