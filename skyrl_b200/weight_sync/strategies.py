"""Trainer->rollout weight transfer strategies (reference: skyrl/backends/skyrl_train/weight_sync/
{transfer_strategy,broadcast_strategy,cuda_ipc_strategy,delta_strategy}.py).

* ``InPlaceStrategy``  - colocated engine reading the trainer's parameter buffer: nothing to move, only a
  version bump (the optimizer's parameter push already updated every rank).
* ``PeerPushStrategy`` - disaggregated engines on other GPUs of the NVSwitch domain: each trainer rank pushes
  its 1/W slice of the flat buffer straight into every engine's peer-mapped buffer with one kernel
  (cast fused), then a device barrier; no rank-0 funnel, no per-chunk handles.
* ``BroadcastStrategy`` - NCCL/gloo broadcast of packed chunks from trainer rank 0 (the measured baseline and
  the CPU path).
* ``DeltaStrategy``    - XOR+compressed delta files for engines that share only a filesystem.
"""

from __future__ import annotations

from typing import Callable, Iterable, List, Optional

import torch
import torch.distributed as dist

from .base import WeightChunk, WeightUpdateRequest


class WeightTransferStrategy:
    name = "base"

    def send(self, chunks: Iterable[WeightChunk]) -> int:
        """Transfer all chunks; returns the number of bytes moved."""
        raise NotImplementedError

    def finish(self) -> None:
        return None


class InPlaceStrategy(WeightTransferStrategy):
    name = "in_place"

    def __init__(self, on_updated: Callable[[], None]):
        self.on_updated = on_updated

    def send(self, chunks=None) -> int:
        self.on_updated()
        return 0


class PeerPushStrategy(WeightTransferStrategy):
    """``dst_ptrs``: device pointers (valid in this process) of every engine's flat bf16 weight buffer."""

    name = "peer"

    def __init__(self, peer_ctx, flat_params: torch.Tensor, dst_ptrs: List[int], rank: int, world: int,
                 on_updated: Optional[Callable[[], None]] = None, barrier_channel: int = 6):
        self.ctx, self.flat, self.dst = peer_ctx, flat_params, list(dst_ptrs)
        self.rank, self.world = rank, world
        self.on_updated = on_updated
        self.channel = barrier_channel

    def send(self, chunks=None, src: Optional[torch.Tensor] = None) -> int:
        n = self.flat.numel()
        shard = n // self.world
        lo = self.rank * shard
        piece = (src if src is not None else self.flat)[lo : lo + shard]
        moved = 0
        for s in range(0, len(self.dst), 8):  # the push kernel fans out to 8 destinations per launch
            self.ctx.push_bf16(piece, self.dst[s : s + 8], dst_offset=lo)
            moved += piece.numel() * 2 * len(self.dst[s : s + 8])
        self.ctx.barrier(self.channel)
        if self.on_updated is not None:
            self.on_updated()
        return moved


class BroadcastStrategy(WeightTransferStrategy):
    """Rank ``src`` of ``group`` broadcasts each packed chunk; receivers hand ``(request, packed)`` to ``on_chunk``."""

    name = "broadcast"

    def __init__(self, group: Optional[dist.ProcessGroup] = None, src: int = 0,
                 on_chunk: Optional[Callable[[WeightUpdateRequest, torch.Tensor], None]] = None, device=None):
        self.group, self.src, self.on_chunk, self.device = group, src, on_chunk, device

    def send(self, chunks: Iterable[WeightChunk]) -> int:
        moved = 0
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        for ch in chunks:
            req = WeightUpdateRequest(ch.names, ch.dtypes, ch.shapes, ch.sizes)
            packed = ch.pack(self.device)
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                meta = [req if rank == self.src else None]
                dist.broadcast_object_list(meta, src=self.src, group=self.group)
                dist.broadcast(packed, src=self.src, group=self.group)
            moved += packed.numel() * packed.element_size()
            if self.on_chunk is not None and rank == self.src:
                self.on_chunk(req, packed)
        return moved

    def receive(self, template_dtype: torch.dtype = torch.bfloat16) -> int:
        """Receiver side of one chunk (ranks other than ``src``); returns bytes received."""
        meta = [None]
        dist.broadcast_object_list(meta, src=self.src, group=self.group)
        req: WeightUpdateRequest = meta[0]
        packed = torch.empty(sum(req.sizes), device=self.device, dtype=template_dtype)
        dist.broadcast(packed, src=self.src, group=self.group)
        if self.on_chunk is not None:
            self.on_chunk(req, packed)
        return packed.numel() * packed.element_size()


def load_chunk_into_model(model, req: WeightUpdateRequest, packed: torch.Tensor) -> None:
    """Receiver helper: slice a packed buffer by ``sizes`` and copy into the fused-layout model by HF name."""
    from ..models import hf_io

    views = hf_io.to_hf_state_dict(model)
    off = 0
    with torch.no_grad():
        for name, shape, n in zip(req.names, req.shapes, req.sizes):
            key = name[len("language_model."):] if name.startswith("language_model.") else name
            dst = views.get(key)
            if dst is None:
                raise KeyError(f"weight '{name}' has no destination in the engine model")
            dst.copy_(packed[off : off + n].view(shape).to(dst.dtype))
            off += n


def select_strategy_name(weight_sync_backend: str, colocate_all: bool, has_peer: bool, delta_cfg=None) -> str:
    """Strategy choice (reference: weight_sync/__init__.py:31-61): delta if configured, in-place / peer when the
    engines are reachable through peer memory, NCCL broadcast otherwise."""
    if delta_cfg is not None or weight_sync_backend == "delta":
        return "delta"
    if colocate_all:
        return "in_place"
    if has_peer and weight_sync_backend in ("nccl", "peer", "ipc"):
        return "peer"
    return "broadcast"
