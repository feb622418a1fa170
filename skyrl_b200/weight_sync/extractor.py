"""Weight extraction from the flat-parameter model: HF-named views, grouped by parent module and batched up to a
byte threshold (reference: weight_sync/weight_extractor_utils.py:11-108, fsdp_worker.py:51-128).  No gather is
needed here -- every rank holds the full bf16 parameter buffer -- so extraction is pure view arithmetic."""

from __future__ import annotations

from typing import Dict, Iterator, List, Tuple

import torch

from ..models import hf_io
from .base import WeightChunk, WeightExtractor


def module_of(name: str) -> str:
    """Parent module of an HF parameter name: the name minus its last two components
    (``model.layers.0.self_attn.q_proj.weight`` -> ``model.layers.0.self_attn``)."""
    parts = name.split(".")
    return ".".join(parts[:-2]) if len(parts) > 2 else name


def group_by_module(named: List[Tuple[str, torch.Tensor]]) -> List[List[Tuple[str, torch.Tensor]]]:
    groups: Dict[str, List[Tuple[str, torch.Tensor]]] = {}
    order: List[str] = []
    for name, t in named:
        m = module_of(name)
        if m not in groups:
            groups[m] = []
            order.append(m)
        groups[m].append((name, t))
    return [groups[m] for m in order]


def batch_groups(groups: List[List[Tuple[str, torch.Tensor]]], threshold_bytes: int) -> Iterator[List[Tuple[str, torch.Tensor]]]:
    """Concatenate module groups into batches of at most ``threshold_bytes`` (a single larger group goes alone)."""
    cur: List[Tuple[str, torch.Tensor]] = []
    cur_b = 0
    for g in groups:
        b = sum(t.numel() * t.element_size() for _, t in g)
        if cur and cur_b + b > threshold_bytes:
            yield cur
            cur, cur_b = [], 0
        cur.extend(g)
        cur_b += b
    if cur:
        yield cur


class FlatModelWeightExtractor(WeightExtractor):
    def __init__(self, model, threshold_gb: float = 1.0, group_by_module: bool = True, name_prefix: str = ""):
        self.model = model
        self.threshold_bytes = int(threshold_gb * (1 << 30))
        self.group = group_by_module
        self.prefix = name_prefix

    def extract_weights(self, dtype: torch.dtype) -> Iterator[WeightChunk]:
        sd = hf_io.to_hf_state_dict(self.model)
        named = [(self.prefix + k, v if v.dtype == dtype else v.to(dtype)) for k, v in sd.items()]
        groups = group_by_module(named) if self.group else [[nt] for nt in named]
        for batch in batch_groups(groups, self.threshold_bytes):
            yield WeightChunk(names=[n for n, _ in batch], dtypes=[str(t.dtype).replace("torch.", "") for _, t in batch],
                              shapes=[list(t.shape) for _, t in batch], tensors=[t.contiguous() for _, t in batch])
