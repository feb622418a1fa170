"""Router replay: record the experts chosen at rollout time and force the same choice in the training forward, so
that train-time and rollout-time log-probabilities of an MoE policy are computed through the same experts.

Reference: skyrl/backends/skyrl_train/utils/replay_utils.py:189-326 and utils/routed_experts.py (the rollout engine
returns ``routed_experts [tokens, layers, top_k]`` per sample; the trainer aligns them with the packed batch and patches
Megatron's TopK router).  Here the MoE layer takes ``routed_indices`` directly (``models/moe.py``); this module holds
the per-forward state: a recorder used by the engine's prefill / decode and a replayer used by the worker.
"""

from __future__ import annotations

import contextlib
import threading
from typing import Dict, List, Optional

import torch

_state = threading.local()


def _get():
    if not hasattr(_state, "mode"):
        _state.mode, _state.store, _state.replay = None, None, None
    return _state


@contextlib.contextmanager
def record_routing():
    """Inside the block every MoE layer appends its ``[T, k]`` expert ids; yields the per-layer list."""
    s = _get()
    prev = (s.mode, s.store)
    s.mode, s.store = "record", {}
    try:
        yield s.store
    finally:
        s.mode, s.store = prev


@contextlib.contextmanager
def replay_routing(indices: torch.Tensor):
    """``indices``: ``[T, layers, k]`` aligned with the packed tokens of the forward run inside the block."""
    s = _get()
    prev = (s.mode, s.replay)
    s.mode, s.replay = "replay", indices
    try:
        yield
    finally:
        s.mode, s.replay = prev


_persistent = {"replay": None}  # process-wide, see set_replay


def set_replay(indices: Optional[torch.Tensor]) -> None:
    """Replay ``indices`` (``[T, layers, k]``) in every forward from now until ``set_replay(None)``.  Unlike the
    ``replay_routing`` block this also covers the layer recomputation that gradient checkpointing runs during the
    backward pass: long after the forward call returned, and on CUDA in the autograd engine's own thread -- which is
    why this state is process-wide while the ``record_routing`` / ``replay_routing`` blocks are per thread."""
    _persistent["replay"] = indices


def active() -> bool:
    """Is any recording or replay in force for the calling thread?"""
    return _get().mode is not None or _persistent["replay"] is not None


PAD = -1  # rows of a replay table without recorded routing: the layer keeps its own choice there


def pad_routes(per_sample: List[Optional[torch.Tensor]], seq_lens: List[int], width: int) -> torch.Tensor:
    """Left-padded ``[B, width, layers, k]`` int16 batch tensor: sample ``i``'s rows sit where its ``seq_lens[i]``
    tokens sit in the left-padded ``sequences`` tensor; tokens that were never routed at rollout time (the final
    sampled token, text appended by the environment after the last model turn) and the padding hold ``PAD``."""
    def as_tensor(t):
        if t is None or isinstance(t, torch.Tensor):
            return t
        import numpy as np

        return torch.from_numpy(np.asarray(t).astype(np.int32))  # wire tables arrive as read-only unsigned arrays

    per_sample = [as_tensor(t) for t in per_sample]
    shape = next((tuple(t.shape[1:]) for t in per_sample if t is not None and t.dim() == 3), None)
    if shape is None:
        raise ValueError("no sample carries routed experts")
    out = torch.full((len(per_sample), width, *shape), PAD, dtype=torch.int16)
    for i, (t, n) in enumerate(zip(per_sample, seq_lens)):
        if t is None:
            continue
        if tuple(t.shape[1:]) != shape:
            raise ValueError(f"sample {i}: routed experts have shape {tuple(t.shape)}, expected [*, {shape[0]}, {shape[1]}]")
        m = min(int(n), t.shape[0])
        out[i, width - int(n) : width - int(n) + m] = t[:m].to(torch.int16)
    return out


def on_route(layer: int, idx: torch.Tensor) -> Optional[torch.Tensor]:
    """Called by the MoE layer with its own top-k choice; returns the indices to use instead (replay) or ``None``."""
    s = _get()
    if s.mode == "record":
        s.store[layer] = idx.detach()
        return None
    if s.mode == "replay" or _persistent["replay"] is not None:
        r = (s.replay if s.mode == "replay" else _persistent["replay"])[:, layer]
        if r.shape != idx.shape:
            raise ValueError(f"replayed routing for layer {layer} has shape {tuple(r.shape)}, expected {tuple(idx.shape)}")
        r = r.to(idx.device).to(idx.dtype)
        return torch.where(r >= 0, r, idx)
    return None


def stack_recorded(store: Dict[int, torch.Tensor]) -> torch.Tensor:
    """Per-layer ``[T, k]`` -> ``[T, layers, k]`` in layer order."""
    return torch.stack([store[i] for i in sorted(store)], dim=1)


def align_to_packed(per_sample: List[torch.Tensor], seq_lens: List[int], pad_value: int = 0) -> torch.Tensor:
    """Concatenate per-sample ``[len_i, L, k]`` tables in packed order; a sample whose table is one row short (the
    last generated token was never fed back through the model) repeats its final row."""
    out = []
    for t, n in zip(per_sample, seq_lens):
        if t.shape[0] < n:
            pad = t[-1:].expand(n - t.shape[0], *t.shape[1:]) if t.shape[0] else torch.full((n, *t.shape[1:]), pad_value, dtype=t.dtype)
            t = torch.cat([t, pad], 0)
        out.append(t[:n])
    return torch.cat(out, 0)
