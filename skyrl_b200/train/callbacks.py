"""Training callbacks: custom behaviour at training events without subclassing a trainer.

Every event method takes the same three arguments, ``(trainer, callback_input, control)``:

* ``trainer``: the ``PPOTrainer`` / ``SFTTrainer``; ``cfg``, ``tracker``, ``tokenizer`` and ``global_step`` are the
  stable surface.
* ``callback_input``: a ``CallbackInput`` snapshot.  The loop counters are always filled; ``batch``, ``metrics``,
  ``logs`` and ``ckpt_path`` only for the events they belong to.
* ``control``: a ``TrainingControl`` whose flags request a checkpoint, an evaluation or (an addition here) a stop.  The
  trainer reads the flags once per step, right after ``on_step_end``, and resets them.

Event names, argument order and dataclass fields are those of the reference (skyrl/train/utils/callbacks.py), so a
callback written for it runs here unchanged.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

EVENTS = ("on_train_start", "on_train_end", "on_epoch_start", "on_epoch_end", "on_step_start", "on_step_end",
          "on_eval_start", "on_eval_end", "on_save", "on_log")


@dataclass
class CallbackInput:
    global_step: int
    epoch: int
    total_steps: int
    steps_per_epoch: int
    batch: Optional[Any] = None               # step events: the training batch
    metrics: Optional[Dict[str, Any]] = None  # step end / eval end
    logs: Optional[Dict[str, Any]] = None     # on_log: the dict about to be committed; may be extended in place
    ckpt_path: Optional[str] = None           # on_save


@dataclass
class TrainingControl:
    should_save: bool = False
    should_evaluate: bool = False
    should_stop: bool = False

    def reset(self) -> None:
        self.should_save = self.should_evaluate = self.should_stop = False


class TrainingCallback:
    """Base class: override the events you need."""

    def on_train_start(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """Once, before the loop (after a checkpoint was resumed)."""

    def on_train_end(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """Once, after the loop and the final saves."""

    def on_epoch_start(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None: ...

    def on_epoch_end(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None: ...

    def on_step_start(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """Before a training step; ``callback_input.batch`` is what the step starts from."""

    def on_step_end(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """After a training step; ``batch`` and ``metrics`` are set.  Set control flags here."""

    def on_eval_start(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None: ...

    def on_eval_end(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """``callback_input.metrics`` holds the evaluation metrics."""

    def on_save(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """After a checkpoint was written to ``callback_input.ckpt_path``."""

    def on_log(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        """Before metrics go to the tracker; extend ``callback_input.logs`` in place to add fields."""


class CallbackHandler(TrainingCallback):
    """Fan-out: itself a callback; calls every registered callback in registration order.  ``fire`` is what trainers
    use: it builds the ``CallbackInput`` from the trainer's counters and hands out the shared ``control``."""

    def __init__(self, callbacks: Optional[List[TrainingCallback]] = None):
        self.callbacks: List[TrainingCallback] = list(callbacks or [])
        self.control = TrainingControl()

    def add(self, callback: TrainingCallback) -> None:
        self.callbacks.append(callback)

    append = add

    def __iter__(self):
        return iter(self.callbacks)

    def __len__(self) -> int:
        return len(self.callbacks)

    def _dispatch(self, name: str, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        for cb in self.callbacks:
            getattr(cb, name)(trainer, callback_input, control)

    def fire(self, event: str, trainer, **fields) -> TrainingControl:
        if event not in EVENTS:
            raise ValueError(f"unknown callback event '{event}'")
        if self.callbacks:
            ci = CallbackInput(global_step=int(getattr(trainer, "global_step", 0)), epoch=int(getattr(trainer, "epoch", 0)),
                               total_steps=int(getattr(trainer, "total_steps", 0) or 0),
                               steps_per_epoch=int(getattr(trainer, "steps_per_epoch", 0) or 0), **fields)
            self._dispatch(event, trainer, ci, self.control)
        return self.control


def _fan_out(name: str):
    def method(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        self._dispatch(name, trainer, callback_input, control)

    method.__name__ = name
    return method


for _name in EVENTS:
    setattr(CallbackHandler, _name, _fan_out(_name))


class EarlyStopOnReward(TrainingCallback):
    """Example: checkpoint and stop once the average reward has passed a threshold ``patience`` steps in a row."""

    def __init__(self, threshold: float, key: str = "reward/avg_raw_reward", patience: int = 1):
        self.threshold, self.key, self.patience, self.hits = threshold, key, patience, 0

    def on_step_end(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        m = callback_input.metrics or {}
        if m.get(self.key, float("-inf")) >= self.threshold:
            self.hits += 1
            if self.hits >= self.patience:
                control.should_save = True
                control.should_stop = True
        else:
            self.hits = 0
