"""Trainer -> engine weight sync across different tensor-parallel layouts, as block copies pushed by the owning rank.

The reference reaches the engine's layout through full tensors: every parameter is all-gathered
(``DTensor.full_tensor()``, skyrl/backends/skyrl_train/workers/fsdp/fsdp_worker.py:125-128; Megatron-Bridge
``export_hf_weights``, workers/megatron/megatron_worker.py:264-328), cast, packed and re-sliced by the engine's loader
(weight_sync/cuda_ipc_strategy.py:206-222).  Here the re-layout is computed once, on the host, as a *plan*: for every
parameter, the rectangle of the full matrix that a trainer shard holds is intersected with the rectangle that each
destination engine shard needs, which yields a list of 2-D block copies "from my flat buffer to that engine's flat
buffer".  One kernel launch per sync (``csrc/weight_sync.cu``) executes the whole list with peer stores, so the fused
QKV / gate-up re-slicing, the TP4 -> TP2 regrouping and the optional fp32 -> bf16 cast all happen in flight.

Sharding convention (``models/tp_decoder.py::shard_param``): fused QKV and gate/up are sliced per component along the
rows, o-proj / down-proj along the columns, everything else is replicated.  A replicated parameter is pushed in
``src_tp`` row chunks, one by each source rank of the group, so the sources share the NVLink load.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.decoder import ModelArgs
from ..ops import _lib

Rect = Tuple[int, int, int, int, int, int]  # full rows [r0, r1), full cols [c0, c1), local row / col of (r0, c0)


def shard_rects(name: str, shape: Tuple[int, ...], a: ModelArgs, tp: int, r: int,
                vocab_parallel_head: bool = False) -> Tuple[List[Rect], Tuple[int, int]]:
    """Rectangles of the full parameter held by shard ``r`` of ``tp`` and the local matrix shape ``(rows, cols)``.
    One-dimensional parameters are treated as one-column matrices."""
    leaf = name.split(".")[-1]
    rows, cols = (shape[0], int(np.prod(shape[1:]))) if len(shape) > 1 else (shape[0], 1)
    if tp == 1:
        return [(0, rows, 0, cols, 0, 0)], (rows, cols)
    if leaf == "lm_head" and vocab_parallel_head:
        vs = rows // tp
        return [(r * vs, (r + 1) * vs, 0, cols, 0, 0)], (vs, cols)
    if leaf in ("wqkv", "bqkv"):
        comps = [a.q_dim, a.kv_dim, a.kv_dim]
    elif leaf == "wgu":
        comps = [a.intermediate_size, a.intermediate_size]
    elif leaf in ("wo", "wd"):
        w = cols // tp
        return [(0, rows, r * w, (r + 1) * w, 0, 0)], (rows, w)
    else:
        return [(0, rows, 0, cols, 0, 0)], (rows, cols)
    rects, base, lbase = [], 0, 0
    for c in comps:
        cs = c // tp
        rects.append((base + r * cs, base + (r + 1) * cs, 0, cols, lbase, 0))
        base += c
        lbase += cs
    return rects, (lbase, cols)


def is_replicated(name: str, tp: int, vocab_parallel_head: bool = False) -> bool:
    leaf = name.split(".")[-1]
    if leaf == "lm_head" and vocab_parallel_head and tp > 1:
        return False
    return tp == 1 or leaf not in ("wqkv", "bqkv", "wgu", "wo", "wd")


@dataclass
class BlockCopy:
    name: str
    dest: int        # index into the destination list
    src_off: int     # element offset in the source flat buffer
    dst_off: int     # element offset in the destination flat buffer
    rows: int
    cols: int        # elements per row
    src_ld: int      # elements between rows at the source
    dst_ld: int


@dataclass
class Destination:
    """One engine shard that receives data: its flat buffer (pointer as seen from the source rank, or a tensor for the
    PyTorch executor), the name -> (offset, numel) table of that buffer, and its position in the engine's TP group."""

    ptr: int
    offsets: Dict[str, Tuple[int, int]]
    tp: int
    rank: int
    tensor: Optional[torch.Tensor] = None


def full_shapes(a: ModelArgs) -> Dict[str, Tuple[int, ...]]:
    from ..models.decoder import _param_specs

    return dict(_param_specs(a))


def build_plan(full_args: ModelArgs, src_offsets: Dict[str, Tuple[int, int]], src_tp: int, src_rank: int,
               dests: Sequence[Destination], names: Optional[Sequence[str]] = None,
               src_vocab_parallel_head: bool = False, chunk_world: int = 1, chunk_rank: int = 0) -> List[BlockCopy]:
    """Block copies that move everything this source shard owns to every destination that needs it.

    ``chunk_world`` / ``chunk_rank``: this source is one of ``chunk_world`` data-parallel replicas that hold the same
    shard; each replica then pushes only its 1 / ``chunk_world`` of every block's rows, so the replicas share the
    link load and nothing is sent twice (disaggregated engines fed by a data-parallel trainer)."""
    shapes = full_shapes(full_args)
    plan: List[BlockCopy] = []
    for name in (names or list(src_offsets)):
        if name not in shapes:
            continue
        shape = shapes[name]
        s_rects, (s_rows, s_cols) = shard_rects(name, shape, full_args, src_tp, src_rank, src_vocab_parallel_head)
        s_base = src_offsets[name][0]
        if is_replicated(name, src_tp, src_vocab_parallel_head) and src_tp > 1:
            # every source rank holds the whole parameter: each pushes one chunk of the rows
            rows = shape[0]
            per = -(-rows // src_tp)
            per = -(-per // 8) * 8  # keep 16-byte alignment for one-dimensional parameters
            lo, hi = min(rows, src_rank * per), min(rows, (src_rank + 1) * per)
            s_rects = [(lo, hi, 0, s_cols, lo, 0)] if hi > lo else []
        if chunk_world > 1:
            cut = []
            for (r0, r1, c0, c1, lr, lc) in s_rects:
                per = -(-(r1 - r0) // chunk_world)
                per = -(-per // 8) * 8
                lo, hi = min(r1, r0 + chunk_rank * per), min(r1, r0 + (chunk_rank + 1) * per)
                if hi > lo:
                    cut.append((lo, hi, c0, c1, lr + (lo - r0), lc))
            s_rects = cut
        for di, d in enumerate(dests):
            if name not in d.offsets:
                continue
            d_rects, (d_rows, d_cols) = shard_rects(name, shape, full_args, d.tp, d.rank)
            d_base = d.offsets[name][0]
            for (sr0, sr1, sc0, sc1, slr, slc) in s_rects:
                for (dr0, dr1, dc0, dc1, dlr, dlc) in d_rects:
                    r0, r1, c0, c1 = max(sr0, dr0), min(sr1, dr1), max(sc0, dc0), min(sc1, dc1)
                    if r1 <= r0 or c1 <= c0:
                        continue
                    so = s_base + (slr + r0 - sr0) * s_cols + (slc + c0 - sc0)
                    do = d_base + (dlr + r0 - dr0) * d_cols + (dlc + c0 - dc0)
                    nrows, ncols = r1 - r0, c1 - c0
                    if ncols == s_cols and ncols == d_cols:  # whole rows on both sides: one contiguous run
                        plan.append(BlockCopy(name, di, so, do, 1, nrows * ncols, nrows * ncols, nrows * ncols))
                    else:
                        plan.append(BlockCopy(name, di, so, do, nrows, ncols, s_cols, d_cols))
    return plan


def run_plan_reference(plan: Sequence[BlockCopy], src_flat: torch.Tensor, dests: Sequence[Destination]) -> None:
    """PyTorch executor of a plan (CPU tests, and the oracle of the kernel)."""
    for c in plan:
        dst = dests[c.dest].tensor
        s = torch.as_strided(src_flat, (c.rows, c.cols), (c.src_ld, 1), c.src_off)
        torch.as_strided(dst, (c.rows, c.cols), (c.dst_ld, 1), c.dst_off).copy_(s.to(dst.dtype))


_DESC = np.dtype([("src", "u8"), ("dst", "u8"), ("ss", "i8"), ("ds", "i8"), ("first", "i8"), ("rows", "i4"), ("vpr", "i4"),
                  ("cast", "i4"), ("pad", "i4")])


class RelayoutPush:
    """A plan compiled to the kernel's descriptor table (kept on the device; re-used for every sync)."""

    def __init__(self, plan: Sequence[BlockCopy], src_flat: torch.Tensor, dests: Sequence[Destination]):
        lib = _lib.kernels()
        lib.sb_relayout_push.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p]
        assert int(lib.sb_relayout_desc_bytes()) == _DESC.itemsize
        per_item = int(lib.sb_relayout_vecs_per_item())
        self.src_flat = src_flat
        cast = src_flat.dtype == torch.float32
        se = src_flat.element_size()
        arr = np.zeros(len(plan), dtype=_DESC)
        items = 0
        self.bytes_out = 0
        for i, c in enumerate(plan):
            if c.cols % 8 or c.src_off % 8 or c.dst_off % 8 or (c.rows > 1 and (c.src_ld % 8 or c.dst_ld % 8)):
                raise ValueError(f"block copy of '{c.name}' is not 16-byte aligned: {c}")
            arr[i] = (src_flat.data_ptr() + c.src_off * se, dests[c.dest].ptr + c.dst_off * 2, c.src_ld * se, c.dst_ld * 2,
                      items, c.rows, c.cols // 8, int(cast), 0)
            items += -(-(c.rows * (c.cols // 8)) // per_item)
            self.bytes_out += c.rows * c.cols * 2
        self.n_desc, self.n_items = len(plan), items
        self.descs = torch.from_numpy(arr.view(np.uint8).copy()).to(src_flat.device) if len(plan) else None

    def run(self) -> None:
        if self.n_desc == 0:
            return
        _lib.check(_lib.kernels().sb_relayout_push(self.descs.data_ptr(), self.n_desc, self.n_items, _lib.stream_ptr()),
                   "sb_relayout_push")
