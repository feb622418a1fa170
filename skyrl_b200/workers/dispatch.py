"""``trainer.dispatch``: the reference's worker verbs by role name, over this package's SPMD workers.

In the reference a driver process owns a ``WorkerDispatch`` that ships batches to actor groups and manages who is on
the GPU (skyrl/backends/skyrl_train/workers/worker_dispatch.py:44-707).  Here every rank *is* a worker of every role,
so there is nothing to ship: a verb is a method call on this rank's worker (collectives inside it line the ranks up).
The facade exists so that trainer subclasses and callbacks written against ``trainer.dispatch.forward("policy", batch)``,
``forward_backward(...)``, ``optim_step(...)``, ``save_weights_for_sampler()`` ... keep working; offload / backload
bookkeeping happens inside the workers' own ``offload`` / ``backload``.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from ..train.batch import TrainingInputBatch, TrainingOutputBatch


class WorkerDispatch:
    ROLES = ("policy", "critic", "ref")

    def __init__(self, trainer):
        self._t = trainer

    # ------------------------------------------------------------------ lookup
    def _worker(self, model: str):
        if model not in self.ROLES:
            raise ValueError(f"unknown model role '{model}'; expected one of {self.ROLES}")
        w = getattr(self._t, model, None)
        if w is None:
            raise ValueError(f"this run has no '{model}' worker")
        return w

    def has(self, model: str) -> bool:
        return model in self.ROLES and getattr(self._t, model, None) is not None

    def dp_size(self, model: str) -> int:
        w = self._worker(model)
        return w.mesh.dp_size if getattr(w, "mesh", None) is not None else w.env.world_size

    def get_lcm_dp_size(self) -> int:
        import math

        sizes = [self.dp_size(m) for m in self.ROLES if self.has(m)]
        return math.lcm(*sizes) if sizes else 1

    # ------------------------------------------------------------------ passes
    def forward(self, model: str, data: TrainingInputBatch, **_unused) -> TrainingOutputBatch:
        return self._worker(model).forward(data)

    def forward_backward(self, model: str, data: TrainingInputBatch, loss_fn: Optional[str] = None,
                         loss_fn_config: Optional[Dict[str, Any]] = None, model_id: Optional[str] = None,
                         **_unused) -> Dict[str, Any]:
        w = self._worker(model)
        if model == "critic":
            return w.forward_backward(data)
        return w.forward_backward(data, loss_fn=loss_fn, loss_fn_config=loss_fn_config)

    def optim_step(self, model: str, model_id: Optional[str] = None) -> Optional[float]:
        return self._worker(model).optim_step()

    def set_lr(self, model: str, learning_rate: float, model_id: Optional[str] = None) -> None:
        self._worker(model).set_lr(float(learning_rate))

    def set_algorithm_config(self, model: str, **kwargs) -> None:
        algo = self._worker(model).cfg.algorithm
        for k, v in kwargs.items():
            if not hasattr(algo, k):
                raise ValueError(f"the algorithm config has no field '{k}'")
            setattr(algo, k, v)

    # ------------------------------------------------------------------ profiling
    def start_profile(self, model: str) -> None:
        self._worker(model).start_profile()

    def profile_step(self, model: str) -> None:
        self._worker(model).profile_step()

    def stop_profile(self, model: str) -> Optional[str]:
        return self._worker(model).stop_profile()

    # ------------------------------------------------------------------ state
    def save_checkpoint(self, model: str, ckpt_dir: str, tokenizer=None, model_id: Optional[str] = None) -> None:
        self._worker(model).save_checkpoint(ckpt_dir)

    def load_checkpoint(self, model: str, ckpt_dir: str, load_optimizer_states: bool = True,
                        load_lr_scheduler_states: bool = True, **_unused) -> None:
        self._worker(model).load_checkpoint(ckpt_dir, load_optimizer_states=load_optimizer_states,
                                            load_lr_scheduler_states=load_lr_scheduler_states)

    def save_hf_model(self, model: str, export_dir: str, tokenizer=None) -> None:
        self._worker(model).save_hf_model(export_dir, tokenizer)

    def offload(self, model: str, offload_optimizer: bool = True, offload_model: bool = True) -> None:
        self._worker(model).offload(include_optimizer=offload_optimizer, include_params=offload_model)

    def backload(self, model: str) -> None:
        self._worker(model).backload()

    def empty_cache(self, model: Optional[str] = None) -> None:
        import torch

        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ weights -> sampler
    def init_weight_sync_state(self, inference_engine_client=None) -> None:
        """Nothing to set up: a colocated engine reads the training buffer (or a copy the worker refreshes) and
        stand-alone servers are reached by the transfer object the trainer already holds."""

    async def save_weights_for_sampler(self, model_id: Optional[str] = None) -> None:
        await self._t.sync_weights_async()

    def get_node_ids(self) -> List[str]:
        import socket

        return [socket.gethostname()]
