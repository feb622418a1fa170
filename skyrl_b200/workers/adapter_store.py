"""Multi-tenant LoRA: many adapters share one resident base model.  Each tenant's adapter parameters, fp32 master
copy and Adam moments live in pinned host memory; ``swap_to`` moves the active tenant's state out and the requested
one in (reference: skyrl/backends/skyrl_train/workers/megatron/adapter_store.py:107-435, ``AdapterStore.swap_to`` with
data-parallel barriers around the swap)."""

from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist


class AdapterSlot:
    def __init__(self, params: torch.Tensor, optimizer, grads: Optional[torch.Tensor] = None) -> None:
        pin = torch.cuda.is_available()

        def host(t: torch.Tensor) -> torch.Tensor:
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
            h.copy_(t)
            return h

        self.params = host(params)
        self.master, self.exp_avg, self.exp_avg_sq = host(optimizer.master), host(optimizer.exp_avg), host(optimizer.exp_avg_sq)
        self.step_count, self.lr = optimizer.step_count, optimizer.lr
        # gradients accumulated by forward_backward calls that no optim_step has consumed yet: a tenant may be swapped
        # out between the two (reference: adapter_store.py:113-125, ``cpu_grad_data``)
        self.grads = host(grads) if grads is not None else None
        self.microbatches = 0


class AdapterStore:
    """Owns the slots of one worker.  The worker's live adapter buffer and optimizer are reused for every tenant."""

    def __init__(self, worker, max_slots: int = 8):
        from ..models.lora import LoRACausalLM

        if not isinstance(worker.model, LoRACausalLM):
            raise ValueError("AdapterStore needs a worker whose model carries LoRA adapters")
        self.worker, self.max_slots = worker, max_slots
        self.slots: Dict[str, AdapterSlot] = {}
        self.active: Optional[str] = None

    def _barrier(self) -> None:
        if dist.is_initialized():
            dist.barrier()

    def _save_active(self) -> None:
        if self.active is None:
            return
        w = self.worker
        s = self.slots[self.active]
        s.params.copy_(w.model.flat_params, non_blocking=True)
        s.master.copy_(w.optimizer.master, non_blocking=True)
        s.exp_avg.copy_(w.optimizer.exp_avg, non_blocking=True)
        s.exp_avg_sq.copy_(w.optimizer.exp_avg_sq, non_blocking=True)
        s.step_count, s.lr = w.optimizer.step_count, w.optimizer.lr
        if s.grads is not None:
            s.grads.copy_(w.flat_grad, non_blocking=True)
            s.microbatches = w.num_microbatches_accumulated
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    def create(self, name: str, seed: int = 0) -> None:
        """New tenant with freshly initialised adapters and zeroed optimizer state; becomes the active one."""
        if name in self.slots:
            raise ValueError(f"adapter '{name}' already exists")
        if len(self.slots) >= self.max_slots:
            raise RuntimeError(f"adapter store is full ({self.max_slots} slots)")
        self._barrier()
        self._save_active()
        w = self.worker
        w.model.reset_lora(seed)
        o = w.optimizer
        o.master.copy_(w.model.flat_params[o.lo : o.lo + o.shard].float())
        o.exp_avg.zero_()
        o.exp_avg_sq.zero_()
        o.step_count = 0
        o.zero_grad()
        w.num_microbatches_accumulated = 0
        self.slots[name] = AdapterSlot(w.model.flat_params, o, getattr(w, "flat_grad", None))
        self.active = name
        self._barrier()

    def swap_to(self, name: str) -> None:
        if name == self.active:
            return
        if name not in self.slots:
            raise KeyError(f"unknown adapter '{name}'")
        self._barrier()
        self._save_active()
        w, s = self.worker, self.slots[name]
        w.model.flat_params.copy_(s.params, non_blocking=True)
        w.optimizer.master.copy_(s.master, non_blocking=True)
        w.optimizer.exp_avg.copy_(s.exp_avg, non_blocking=True)
        w.optimizer.exp_avg_sq.copy_(s.exp_avg_sq, non_blocking=True)
        w.optimizer.step_count, w.optimizer.lr = s.step_count, s.lr
        w.optimizer.zero_grad()
        w.num_microbatches_accumulated = 0
        if s.grads is not None:
            w.flat_grad.copy_(s.grads, non_blocking=True)
            w.num_microbatches_accumulated = s.microbatches
        self.active = name
        w.refresh_engine_model()
        self._barrier()

    def delete(self, name: str) -> None:
        self.slots.pop(name)
        if self.active == name:
            self.active = None
