"""``TensorBatch`` / ``TrainingInputBatch``: a dict of tensors sharing a leading batch dimension.

Same role and key schema as the reference container (skyrl/backends/skyrl_train/training_batch.py:121-503):
``sequences, attention_mask, response_mask, loss_mask, rewards, rollout_logprobs, action_log_probs,
base_action_log_probs, values, returns, advantages, ...`` plus a free-form ``metadata`` dict.  Batches
never cross a process boundary on the hot path here (each rank builds its own shard), so there is no
custom pickling; ``to_bytes`` / ``from_bytes`` exist for the API server and checkpoints.
"""

from __future__ import annotations

import io
from typing import Any, Dict, Iterator, List, Optional, Sequence

import torch

TRAINING_INPUT_KEYS = (
    "sequences", "attention_mask", "response_mask", "loss_mask", "rewards", "rollout_logprobs", "action_log_probs",
    "base_action_log_probs", "values", "returns", "advantages", "rollout_expert_indices", "router_padding_mask",
    "pixel_values", "image_grid_thw", "kl",
)  # fmt: skip


class TensorList:
    """A batch column whose rows are tensors of different shapes (image patches per sample): supports the same
    batch-dimension operations as a tensor column (reference: ``TensorList`` in training_batch.py:40-118)."""

    def __init__(self, tensors: Sequence[torch.Tensor]):
        self.tensors: List[torch.Tensor] = list(tensors)

    @property
    def shape(self):
        return (len(self.tensors),)

    def __len__(self) -> int:
        return len(self.tensors)

    def __iter__(self):
        return iter(self.tensors)

    def __getitem__(self, idx):
        if isinstance(idx, int):
            return self.tensors[idx]
        if isinstance(idx, slice):
            return TensorList(self.tensors[idx])
        if isinstance(idx, torch.Tensor):
            idx = idx.tolist()
        return TensorList([self.tensors[int(i)] for i in idx])

    @property
    def is_cuda(self) -> bool:
        return bool(self.tensors) and self.tensors[0].is_cuda

    @property
    def device(self):
        return self.tensors[0].device if self.tensors else torch.device("cpu")

    def is_floating_point(self) -> bool:
        return bool(self.tensors) and self.tensors[0].is_floating_point()

    def to(self, *a, **k) -> "TensorList":
        return TensorList([t.to(*a, **k) for t in self.tensors])

    def cpu(self) -> "TensorList":
        return TensorList([t.cpu() for t in self.tensors])

    def contiguous(self) -> "TensorList":
        return TensorList([t.contiguous() for t in self.tensors])

    def pin_memory(self) -> "TensorList":
        return TensorList([t.pin_memory() for t in self.tensors])

    def repeat_interleave(self, times: int, dim: int = 0) -> "TensorList":
        return TensorList([t for t in self.tensors for _ in range(times)])

    @staticmethod
    def cat(lists: Sequence["TensorList"]) -> "TensorList":
        return TensorList([t for l in lists for t in l.tensors])

    def flat(self) -> torch.Tensor:
        """All rows concatenated along dim 0 (what a vision tower consumes)."""
        return torch.cat(self.tensors, 0) if self.tensors else torch.empty(0)


def _batched(v) -> bool:
    return isinstance(v, (torch.Tensor, TensorList))


class TensorBatch(dict):
    """dict[str, Tensor | None] with batch-dimension operations. ``None`` values are carried through."""

    def __init__(self, *args, metadata: Optional[Dict[str, Any]] = None, **kwargs):
        super().__init__(*args, **kwargs)
        self.metadata: Dict[str, Any] = dict(metadata or {})
        self._check()

    # ------------------------------------------------------------------ invariants
    def _check(self) -> None:
        sizes = {k: v.shape[0] for k, v in self.items() if _batched(v)}
        if len(set(sizes.values())) > 1:
            raise ValueError(f"batch size mismatch across keys: {sizes}")

    @property
    def batch_size(self) -> int:
        for v in self.values():
            if _batched(v):
                return v.shape[0]
        return 0

    def __len__(self) -> int:  # number of rows, like the reference container
        return self.batch_size

    @property
    def device(self):
        for v in self.values():
            if isinstance(v, torch.Tensor):
                return v.device
        return None

    def __setitem__(self, key, value):
        if _batched(value) and self.batch_size and len(self.keys() - {key}) and \
                value.shape[0] != self.batch_size:
            raise ValueError(f"'{key}' has batch size {value.shape[0]}, expected {self.batch_size}")
        super().__setitem__(key, value)

    # ------------------------------------------------------------------ batch ops
    def _map(self, fn) -> "TensorBatch":
        out = type(self)({k: (fn(v) if _batched(v) else v) for k, v in self.items()},
                         metadata=dict(self.metadata))
        return out

    def to(self, device=None, dtype=None, non_blocking: bool = False) -> "TensorBatch":
        def mv(t):
            if dtype is not None and t.is_floating_point():
                return t.to(device=device, dtype=dtype, non_blocking=non_blocking)
            return t.to(device=device, non_blocking=non_blocking)

        return self._map(mv)

    def pin_memory(self) -> "TensorBatch":
        return self._map(lambda t: t.pin_memory() if not t.is_cuda and torch.cuda.is_available() else t)

    def contiguous(self) -> "TensorBatch":
        return self._map(lambda t: t.contiguous())

    def slice(self, start: int, end: int) -> "TensorBatch":
        return self._map(lambda t: t[start:end])

    def select(self, index) -> "TensorBatch":
        idx = torch.as_tensor(index, dtype=torch.long)
        return self._map(lambda t: t[idx.to(t.device)])

    def chunk(self, chunk_size: int) -> List["TensorBatch"]:
        """Split into consecutive pieces of ``chunk_size`` rows (the last may be shorter)."""
        n = self.batch_size
        return [self.slice(s, min(n, s + chunk_size)) for s in range(0, n, chunk_size)]

    def split_equal(self, parts: int) -> List["TensorBatch"]:
        n = self.batch_size
        if n % parts != 0:
            raise ValueError(f"batch size {n} is not divisible by {parts}")
        return self.chunk(n // parts)

    def repeat(self, times: int) -> "TensorBatch":
        return self._map(lambda t: t.repeat_interleave(times, dim=0))

    @classmethod
    def cat(cls, batches: Sequence["TensorBatch"]) -> "TensorBatch":
        if not batches:
            raise ValueError("cannot concatenate an empty list of batches")
        keys = list(batches[0].keys())
        out = {}
        for k in keys:
            vals = [b[k] for b in batches]
            if all(v is None for v in vals):
                out[k] = None
            elif any(v is None for v in vals):
                raise ValueError(f"key '{k}' is None in some batches but not all")
            elif isinstance(vals[0], TensorList):
                out[k] = TensorList.cat(vals)
            else:
                out[k] = torch.cat(vals, dim=0)
        return cls(out, metadata=dict(batches[0].metadata))

    def iter_rows(self) -> Iterator[Dict[str, Any]]:
        for i in range(self.batch_size):
            yield {k: (v[i] if _batched(v) else v) for k, v in self.items()}

    # ------------------------------------------------------------------ serialisation
    def to_bytes(self) -> bytes:
        buf = io.BytesIO()
        torch.save({"tensors": {k: (v.cpu() if _batched(v) else v) for k, v in self.items()},
                    "metadata": self.metadata}, buf)
        return buf.getvalue()

    @classmethod
    def from_bytes(cls, data: bytes) -> "TensorBatch":
        d = torch.load(io.BytesIO(data), weights_only=False)
        return cls(d["tensors"], metadata=d["metadata"])


class TrainingInputBatch(TensorBatch):
    """Batch handed to the workers; see ``TRAINING_INPUT_KEYS``."""


class TrainingOutputBatch(TensorBatch):
    """Batch returned by ``forward`` (key ``output``)."""


def pad_training_input_batch(batch: TrainingInputBatch, multiple: int) -> TrainingInputBatch:
    """Append copies of the last row with ``loss_mask = 0`` until the size divides ``multiple``.

    The number of added rows is recorded in ``metadata['pad_size']`` (reference: training_batch.py:506-570).
    """
    n = batch.batch_size
    pad = (-n) % multiple
    if pad == 0:
        batch.metadata.setdefault("pad_size", 0)
        return batch
    extra = batch.slice(n - 1, n).repeat(pad)
    for key in ("loss_mask", "response_mask"):
        if extra.get(key) is not None and key == "loss_mask":
            extra[key] = torch.zeros_like(extra[key])
    out = TrainingInputBatch.cat([batch, extra])
    out.metadata = dict(batch.metadata)
    out.metadata["pad_size"] = pad
    if "uids" in out.metadata and out.metadata["uids"] is not None:
        out.metadata["uids"] = list(out.metadata["uids"]) + [f"__pad_{i}" for i in range(pad)]
    return out
