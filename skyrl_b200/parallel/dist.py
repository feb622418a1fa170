"""Process-group bootstrap and mesh helpers: one process per GPU, NCCL for CUDA tensors and gloo for
host objects (the reference initialises ``cpu:gloo,cuda:nccl`` the same way,
skyrl/backends/skyrl_train/workers/worker.py:118-143).  Everything degrades to a single process when
``WORLD_SIZE`` is unset, and to gloo-only on machines without a GPU.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistEnv:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    device: torch.device = torch.device("cpu")

    @property
    def is_main(self) -> bool:
        return self.rank == 0


_ENV: Optional[DistEnv] = None


def init_distributed(backend: Optional[str] = None, timeout_s: Optional[int] = None, device: Optional[str] = None) -> DistEnv:
    """Initialise ``torch.distributed`` from the torchrun environment variables (idempotent)."""
    global _ENV
    if _ENV is not None:
        return _ENV
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and device != "cpu"
    dev = torch.device(f"cuda:{local}") if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
        if os.environ.get("SKYRL_B200_NUMA_PIN", "1") not in ("0", "false", "False"):
            try:  # host threads (input staging, scheduler) next to the GPU; silently skipped without sysfs topology
                from ..utils.numa import pin_to_gpu_numa_node

                pin_to_gpu_numa_node(local)
            except Exception:
                pass
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "cpu:gloo,cuda:nccl" if use_cuda else "gloo"
        if timeout_s is None:
            timeout_s = int(os.environ.get("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", "600"))
        kw = {}
        if use_cuda:
            kw["device_id"] = dev
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    _ENV = DistEnv(rank, local, world, dev)
    return _ENV


@dataclass
class ParallelMesh:
    """(dp, tp) factorisation of the world: tensor-parallel groups are runs of ``tp`` consecutive ranks (they share
    NVLink peers), data-parallel groups take every ``tp``-th rank."""

    tp_size: int = 1
    dp_size: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    tp_cpu_group: Optional[object] = None  # gloo-only twin of tp_group for host-side object exchange


_MESHES: dict = {}


def build_mesh(tp: int, env: Optional[DistEnv] = None) -> ParallelMesh:
    """Create (once per ``tp``) the process groups of a ``dp x tp`` mesh. Collective: every rank must call it."""
    env = env or get_env()
    if tp in _MESHES:
        return _MESHES[tp]
    W, r = env.world_size, env.rank
    if tp < 1 or W % tp != 0:
        raise ValueError(f"tensor parallel size {tp} does not divide the world size {W}")
    mesh = ParallelMesh(tp, W // tp, r % tp, r // tp)
    if W > 1 and dist.is_initialized():
        for g in range(W // tp):  # every rank creates every group, in the same order
            ranks = list(range(g * tp, (g + 1) * tp))
            grp = dist.new_group(ranks)
            cpu = dist.new_group(ranks, backend="gloo")
            if r in ranks:
                mesh.tp_group = grp
                mesh.tp_cpu_group = cpu
        for t in range(tp):
            ranks = list(range(t, W, tp))
            grp = dist.new_group(ranks)
            if r in ranks:
                mesh.dp_group = grp
    _MESHES[tp] = mesh
    return mesh


_HSDP: dict = {}


def build_hsdp_groups(fsdp_size: int, env: Optional[DistEnv] = None):
    """``(shard_group, replica_group)`` of a hybrid-sharded layout: runs of ``fsdp_size`` consecutive ranks shard the
    optimizer state among themselves; ranks with the same position in different runs are replicas of each other.
    Collective: every rank must call it (reference mesh: skyrl/backends/skyrl_train/distributed/fsdp_utils.py:254-261)."""
    env = env or get_env()
    if fsdp_size in _HSDP:
        return _HSDP[fsdp_size]
    W, r = env.world_size, env.rank
    if fsdp_size < 1 or W % fsdp_size != 0:
        raise ValueError(f"fsdp_size {fsdp_size} does not divide the world size {W}")
    shard = replica = None
    if W > 1 and dist.is_initialized():
        for g in range(W // fsdp_size):
            ranks = list(range(g * fsdp_size, (g + 1) * fsdp_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                shard = grp
        for t in range(fsdp_size):
            ranks = list(range(t, W, fsdp_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                replica = grp
    _HSDP[fsdp_size] = (shard, replica)
    return _HSDP[fsdp_size]


def get_env() -> DistEnv:
    return _ENV if _ENV is not None else init_distributed()


def reset_env_for_tests() -> None:
    global _ENV
    _ENV = None


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def all_reduce_max_scalar(x: float, device) -> float:
    """MAX over ranks of a host scalar (used for device-timed step durations)."""
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_reduce_sum_scalar(x: float, device) -> float:
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def shutdown() -> None:
    global _ENV
    if dist.is_initialized():
        dist.destroy_process_group()
    _ENV = None
    _MESHES.clear()
    _HSDP.clear()
