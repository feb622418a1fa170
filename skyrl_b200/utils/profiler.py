"""Profiling helpers: a scheduled ``torch.profiler`` wrapper for selected ranks, a CUDA-event timer, and
device-side step timing reduced with MAX over ranks (reference: skyrl/backends/skyrl_train/utils/profiler.py:22-143)."""

from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch


class Profiler:
    def __init__(self, cfg, rank: int = 0):
        """``cfg``: a ``TorchProfilerConfig``. Inactive unless ``enable`` and this rank is listed."""
        self.cfg = cfg
        self.rank = rank
        self.active = bool(cfg.enable) and rank in list(cfg.ranks)
        self.prof = None
        self.last_summary: Optional[str] = None
        if not self.active:
            return
        acts = []
        if "cpu" in [str(a).lower() for a in cfg.activities]:
            acts.append(torch.profiler.ProfilerActivity.CPU)
        if "cuda" in [str(a).lower() for a in cfg.activities] and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.save_path = cfg.save_path or "/tmp/skyrl-profiles"
        os.makedirs(self.save_path, exist_ok=True)
        sched = torch.profiler.schedule(skip_first=cfg.skip_first, wait=cfg.wait, warmup=cfg.warmup, active=cfg.active,
                                        repeat=cfg.repeat)
        self.prof = torch.profiler.profile(activities=acts, schedule=sched, on_trace_ready=self._on_ready,
                                           record_shapes=cfg.record_shapes, profile_memory=cfg.profile_memory,
                                           with_stack=cfg.with_stack, with_flops=cfg.with_flops,
                                           with_modules=cfg.with_modules)

    def _on_ready(self, prof) -> None:
        tag = f"rank{self.rank}_step{prof.step_num}"
        if self.cfg.export_type == "stacks":
            prof.export_stacks(os.path.join(self.save_path, f"{tag}.stacks"), "self_cuda_time_total")
        else:
            prof.export_chrome_trace(os.path.join(self.save_path, f"{tag}.json"))
        try:
            self.last_summary = prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=25)
        except Exception:
            self.last_summary = None

    def start(self) -> None:
        if self.prof is not None:
            self.prof.start()

    def step(self) -> None:
        if self.prof is not None:
            self.prof.step()

    def stop(self) -> None:
        if self.prof is not None:
            self.prof.stop()

    def kernel_summary(self) -> Optional[str]:
        return self.last_summary


class CudaTimer:
    def __init__(self):
        self.times_ms: Dict[str, List[float]] = {}
        self._open = {}

    def start(self, name: str) -> None:
        s = torch.cuda.Event(enable_timing=True)
        s.record()
        self._open[name] = s

    def stop(self, name: str) -> float:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        e.synchronize()
        ms = self._open.pop(name).elapsed_time(e)
        self.times_ms.setdefault(name, []).append(ms)
        return ms


def device_time_max_over_ranks(ms: float, device) -> float:
    """MAX over ranks of a device-timed duration (the number every multi-GPU report uses)."""
    import torch.distributed as dist

    if not dist.is_initialized():
        return ms
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def start_memory_history(max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def dump_memory_snapshot(path: str) -> None:
    if torch.cuda.is_available():
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        torch.cuda.memory._dump_snapshot(path)
