"""SFT with user callbacks: a perplexity logger and a stop-at-target-loss rule.

A callback sees the trainer and the step's metrics and can ask for a checkpoint, an evaluation or a stop through the
``control`` object; nothing in the trainer has to change.
"""

import math
import sys

from skyrl_b200.config.sft_config import SFTConfig
from skyrl_b200.parallel import dist as pdist
from skyrl_b200.train.callbacks import TrainingCallback
from skyrl_b200.train.sft_trainer import SFTTrainer


class PerplexityLogger(TrainingCallback):
    """Adds exp(loss) to what goes to the tracker and prints a running minimum on the main rank."""

    def __init__(self):
        self.best = float("inf")

    def on_log(self, trainer, callback_input, control):
        logs = callback_input.logs or {}
        if "train/loss" not in logs:
            return
        ppl = math.exp(min(20.0, float(logs["train/loss"])))
        logs["train/perplexity"] = ppl  # in place: the trainer commits this dict
        self.best = min(self.best, ppl)
        if trainer.env.is_main:
            print(f"[callback] step {callback_input.global_step}/{callback_input.total_steps}: perplexity {ppl:.3f} "
                  f"(best {self.best:.3f})", flush=True)


class StopAtLoss(TrainingCallback):
    def __init__(self, target: float):
        self.target = target

    def on_step_end(self, trainer, callback_input, control):
        m = callback_input.metrics or {}
        if float(m.get("train/loss", float("inf"))) <= self.target:
            control.should_save = True
            control.should_stop = True

    def on_save(self, trainer, callback_input, control):
        if trainer.env.is_main:
            print(f"[callback] checkpoint written to {callback_input.ckpt_path}", flush=True)


if __name__ == "__main__":
    cfg = SFTConfig.from_cli_overrides(sys.argv[1:])
    env = pdist.init_distributed()
    try:
        trainer = SFTTrainer(cfg, env=env).setup()
        trainer.add_callback(PerplexityLogger())
        trainer.add_callback(StopAtLoss(target=0.05))
        trainer.train()
    finally:
        pdist.shutdown()
