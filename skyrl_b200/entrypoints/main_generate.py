"""Evaluation-only run: build the policy and its colocated engine, generate over the validation set, report
metrics (reference: skyrl/train/entrypoints/main_generate.py:22-54).

    python -m skyrl_b200.entrypoints.main_generate data.val_data='["val.jsonl"]' trainer.policy.model.path=...
"""

from __future__ import annotations

import json
import sys
from typing import List, Optional

from ..config.config import SkyRLTrainConfig
from ..parallel import dist as pdist
from ..train.dataset import PromptDataset
from .main_base import BasePPOExp


class EvalOnlyEntrypoint(BasePPOExp):
    def get_train_dataset(self):
        return None  # nothing is trained

    def get_eval_dataset(self) -> PromptDataset:
        if not self.cfg.data.val_data:
            raise ValueError("evaluation needs data.val_data")
        return PromptDataset(self.cfg.data.val_data, self.tokenizer, self.cfg.trainer.max_prompt_length)

    def run(self) -> dict:
        try:
            trainer = self._setup_trainer()
            metrics = trainer.eval()
            if trainer.tracker is not None:
                trainer.tracker.log(metrics, 0)
                trainer.tracker.finish()
            if self.env.is_main:
                print(json.dumps(metrics, sort_keys=True))
            return metrics
        finally:
            pdist.shutdown()


def eval_entrypoint(cfg: SkyRLTrainConfig) -> dict:
    return EvalOnlyEntrypoint(cfg).run()


def main(argv: Optional[List[str]] = None) -> None:
    cfg = SkyRLTrainConfig.from_cli_overrides(sys.argv[1:] if argv is None else argv)
    eval_entrypoint(cfg)


if __name__ == "__main__":
    main()
