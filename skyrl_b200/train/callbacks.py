"""Training callbacks in the HF style: event hooks plus a ``TrainingControl`` object through which a
callback can request a checkpoint, an evaluation or a stop (reference: skyrl/train/utils/callbacks.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional


@dataclass
class TrainingControl:
    should_save: bool = False
    should_evaluate: bool = False
    should_stop: bool = False

    def reset(self) -> None:
        self.should_save = self.should_evaluate = self.should_stop = False


class TrainingCallback:
    def on_train_begin(self, trainer, control: Optional[TrainingControl] = None) -> None: ...
    def on_train_end(self, trainer, control: Optional[TrainingControl] = None) -> None: ...
    def on_epoch_begin(self, trainer, epoch: int = 0, control: Optional[TrainingControl] = None) -> None: ...
    def on_epoch_end(self, trainer, epoch: int = 0, control: Optional[TrainingControl] = None) -> None: ...
    def on_step_begin(self, trainer, control: Optional[TrainingControl] = None) -> None: ...
    def on_step_end(self, trainer, metrics: Optional[Dict[str, Any]] = None, control: Optional[TrainingControl] = None) -> None: ...
    def on_generate_end(self, trainer, generator_output=None, control: Optional[TrainingControl] = None) -> None: ...
    def on_evaluate(self, trainer, metrics: Optional[Dict[str, Any]] = None, control: Optional[TrainingControl] = None) -> None: ...
    def on_save(self, trainer, path: str = "", control: Optional[TrainingControl] = None) -> None: ...


class CallbackHandler:
    """Fans events out to callbacks and merges their control requests."""

    def __init__(self, callbacks: Optional[List[TrainingCallback]] = None):
        self.callbacks = list(callbacks or [])
        self.control = TrainingControl()

    def add(self, cb: TrainingCallback) -> None:
        self.callbacks.append(cb)

    def fire(self, event: str, trainer, **kw) -> TrainingControl:
        for cb in self.callbacks:
            fn = getattr(cb, event, None)
            if fn is not None:
                fn(trainer, control=self.control, **kw)
        return self.control


class EarlyStopOnReward(TrainingCallback):
    """Example callback: stop when the running average reward passes a threshold."""

    def __init__(self, threshold: float, key: str = "reward/avg_raw_reward", patience: int = 1):
        self.threshold, self.key, self.patience, self.hits = threshold, key, patience, 0

    def on_step_end(self, trainer, metrics=None, control=None):
        if metrics and metrics.get(self.key, float("-inf")) >= self.threshold:
            self.hits += 1
            if self.hits >= self.patience and control is not None:
                control.should_save = True
                control.should_stop = True
        else:
            self.hits = 0
