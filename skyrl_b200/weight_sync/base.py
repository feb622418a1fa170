"""Weight-sync data types (reference: skyrl/backends/skyrl_train/weight_sync/base.py:10-106).

A ``WeightChunk`` carries full (unsharded) tensors under their HF names, grouped so that tensors a fused
loader needs together (q/k/v, gate/up) travel in one chunk, bounded by a byte threshold.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional

import torch


@dataclass
class WeightChunk:
    names: List[str]
    dtypes: List[str]
    shapes: List[List[int]]
    tensors: List[torch.Tensor]
    module_name: Optional[str] = None
    total_numel: int = field(init=False)
    total_size_bytes: int = field(init=False)

    def __post_init__(self):
        n = len(self.names)
        if not (len(self.dtypes) == len(self.shapes) == len(self.tensors) == n):
            raise ValueError("WeightChunk: names, dtypes, shapes and tensors must have the same length")
        self.total_numel = sum(int(t.numel()) for t in self.tensors)
        self.total_size_bytes = sum(int(t.numel()) * t.element_size() for t in self.tensors)

    def __len__(self) -> int:
        return len(self.names)

    @property
    def sizes(self) -> List[int]:
        return [int(t.numel()) for t in self.tensors]

    def pack(self, device=None) -> torch.Tensor:
        """All tensors flattened into one contiguous buffer (receivers slice it by ``sizes``)."""
        dev = device or (self.tensors[0].device if self.tensors else "cpu")
        dt = self.tensors[0].dtype if self.tensors else torch.bfloat16
        out = torch.empty(self.total_numel, device=dev, dtype=dt)
        off = 0
        for t in self.tensors:
            n = t.numel()
            out[off : off + n].copy_(t.reshape(-1))
            off += n
        return out

    @classmethod
    def unpack(cls, names, dtypes, shapes, packed: torch.Tensor) -> "WeightChunk":
        tensors, off = [], 0
        for shp in shapes:
            n = 1
            for s in shp:
                n *= s
            tensors.append(packed[off : off + n].view(shp))
            off += n
        return cls(list(names), list(dtypes), [list(s) for s in shapes], tensors)


@dataclass
class WeightUpdateRequest:
    names: List[str]
    dtypes: List[str]
    shapes: List[List[int]]
    sizes: Optional[List[int]] = None
    extras: Optional[Dict[str, Any]] = None
    weight_version: Optional[int] = None

    def __len__(self) -> int:
        return len(self.names)


@dataclass
class LoraLoadRequest:
    lora_path: str
    lora_name: str = "skyrl-lora"
    lora_id: int = 1


class WeightExtractor:
    """Yields ``WeightChunk`` objects from a training model in the rollout dtype."""

    def extract_weights(self, dtype: torch.dtype) -> Iterator[WeightChunk]:
        raise NotImplementedError
