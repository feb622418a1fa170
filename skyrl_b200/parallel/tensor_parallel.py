"""Tensor parallelism with sequence-parallel activations, collectives fused into the GEMM kernels.

What the reference gets from Megatron-core / TransformerEngine (``ColumnParallelLinear`` = all-gather -> GEMM,
``RowParallelLinear`` = GEMM -> reduce-scatter, enabled by ``tensor_model_parallel_size`` and
``sequence_parallel = tp > 1``; skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:468-474) is done here by
one kernel per linear layer over NVLink peer memory (``csrc/gemm_tcgen05.cu``, GATHER / SCATTER modes):

* column-parallel forward ``y[:, shard] = all_gather(x) @ W_shard^T``: copy warps inside the GEMM pull the other
  ranks' sequence shards into a local buffer piece by piece while the tensor cores already work on the local shard;
* row-parallel forward ``y = reduce_scatter(x_shard @ W_shard^T)``: the epilogue stores each finished tile directly
  into the owning rank's memory (one slot per source rank); the consumer sums the slots (``reduce_slots`` or the
  fused residual + RMSNorm kernel);
* the backward passes are the same two kernels with the weight read in the other orientation.

Without CUDA peers (CPU tests, gloo) the same functions run a ``torch.distributed`` reference implementation so the
layer logic is testable anywhere.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from .peer import PeerContext, SymmTensor

_cfg = False


def _k():
    global _cfg
    lib = _lib.kernels()
    if not _cfg:
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.sb_gemm_tp.argtypes = [vp, vp, vp, vp, ci, ci, ci, cl, cl, cl, ci, ci, ci, ci, vp, vp, ci, ci, ci, cl, vp, ci, vp]
        lib.sb_gemm_tp_scatter_splitk.argtypes = [vp, vp, ci, ci, ci, cl, cl, vp, ci, ci, cl, ci, vp]
        _cfg = True
    return lib


class TPGroup:
    """Ranks of one tensor-parallel group plus their symmetric work buffers."""

    def __init__(self, peer_ctx: Optional[PeerContext] = None, group: Optional[dist.ProcessGroup] = None,
                 size: Optional[int] = None):
        self.group = group
        if size == 1:  # a trivial group inside a larger world
            self.size, self.rank = 1, 0
        else:
            self.size = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.peer = peer_ctx
        self._gather_bufs = {}
        self._slot_bufs = {}
        self._flags = None

    @property
    def fused(self) -> bool:
        return self.peer is not None and self.size > 1

    # ------------------------------------------------------------------ symmetric buffers
    def gather_buffer(self, rows_total: int, cols: int, tag: str = "x") -> SymmTensor:
        """Full ``[rows_total, cols]`` bf16 activation buffer; rank r writes its shard at rows ``[r*R, (r+1)*R)``."""
        key = (tag, rows_total, cols)
        if key not in self._gather_bufs:
            st = self.peer.alloc(rows_total * cols, torch.bfloat16)
            self._gather_bufs[key] = st
        return self._gather_bufs[key]

    def slot_buffer(self, rows: int, cols: int, dtype: torch.dtype, tag: str = "y") -> SymmTensor:
        """``[size, rows, cols]`` partial-sum slots, slot s written by rank s."""
        key = (tag, rows, cols, dtype)
        if key not in self._slot_bufs:
            self._slot_bufs[key] = self.peer.alloc(self.size * rows * cols, dtype)
        return self._slot_bufs[key]

    def flags(self, m_blocks: int) -> torch.Tensor:
        if self._flags is None or self._flags.numel() < m_blocks + 1:
            self._flags = torch.zeros(max(1024, m_blocks + 1), dtype=torch.int32, device=self.peer.device)
        return self._flags


def gemm_all_gather(tp: TPGroup, x_full: SymmTensor, rows_per_rank: int, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                    w_is_kn: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``all_gather(x) @ W^T`` (or ``@ W`` when ``w_is_kn``) with the gather fused into the GEMM.

    ``x_full.local`` is the ``[size * rows_per_rank, K]`` buffer whose own shard has been written by this rank (and
    a ``tp.peer.barrier()`` passed since, so every rank's shard is complete).  On return the buffer holds all shards,
    which the backward pass needs for the weight gradient anyway."""
    M = tp.size * rows_per_rank
    K = x_full.local.numel() // M
    N = w.shape[1] if w_is_kn else w.shape[0]
    xf = x_full.local.view(M, K)
    if out is None:
        out = torch.empty((M, N), device=xf.device, dtype=torch.bfloat16)
    esz = 2
    peers = (ctypes.c_void_p * tp.size)(*[x_full.ptrs[r] + r * rows_per_rank * K * esz for r in range(tp.size)])
    flags = tp.flags((M + 127) // 128)
    code = _k().sb_gemm_tp(xf.data_ptr(), w.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(), M, N, K,
                           K, w.stride(0), out.stride(0), int(w_is_kn), 0 if out.dtype == torch.bfloat16 else 1, 1, 0,
                           peers, None, tp.size, tp.rank, rows_per_rank, 0, flags.data_ptr(), 0, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_tp(gather)")
    return out


def gemm_reduce_scatter(tp: TPGroup, x: torch.Tensor, w: torch.Tensor, slots: SymmTensor, rows_per_rank: int,
                        w_is_kn: bool = False, all_ranks: bool = False) -> None:
    """``x_shard @ W_shard^T`` whose tiles are stored straight into the owning rank's ``slots`` (slot = this rank).

    With ``all_ranks`` every rank receives all rows (all-reduce layout, ``slots`` is ``[size, M, N]`` on each rank),
    otherwise rank d receives rows ``[d*rows_per_rank, (d+1)*rows_per_rank)`` (``slots`` is ``[size, rows_per_rank, N]``).
    A ``tp.peer.barrier()`` must pass before the slots are read."""
    M, K = x.shape
    N = w.shape[1] if w_is_kn else w.shape[0]
    rows = M if all_ranks else rows_per_rank
    outs = (ctypes.c_void_p * tp.size)(*slots.ptrs)
    out_fp32 = slots.local.dtype == torch.float32
    code = _k().sb_gemm_tp(x.data_ptr(), w.data_ptr(), None, None, M, N, K, x.stride(0), w.stride(0), N, int(w_is_kn),
                           1 if out_fp32 else 0, 0, 2 if all_ranks else 1, None, outs, tp.size, tp.rank,
                           rows_per_rank if not all_ranks else M, rows * N, None, 0, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_tp(scatter)")


def plan_scatter_splitk(M: int, N: int, K: int, n_sm: int = 148) -> int:
    """k slices for a skinny row-parallel projection so that (tiles x slices) covers the SMs (128-wide N tiles)."""
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    k_blocks = (K + 63) // 64
    if tiles >= n_sm or k_blocks < 8:
        return 1
    splits = max(1, min(n_sm // tiles, k_blocks // 4))
    kpb = (k_blocks + splits - 1) // splits
    return (k_blocks + kpb - 1) // kpb  # no empty slice


def gemm_all_reduce_partials(tp: "TPGroup", x: torch.Tensor, w: torch.Tensor, slots: SymmTensor, splits: int) -> None:
    """``x_local @ W_shard^T`` as ``splits`` fp32 k-slice partials stored into slots ``[rank * splits, (rank + 1) *
    splits)`` of *every* rank's ``[size * splits, M, N]`` buffer (decode path of tensor-parallel engines).  A
    ``tp.peer`` barrier must pass before the slots are read."""
    M, K = x.shape
    N = w.shape[0]
    outs = (ctypes.c_void_p * tp.size)(*slots.ptrs)
    code = _k().sb_gemm_tp_scatter_splitk(x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), outs, tp.size,
                                          tp.rank, M * N, splits, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_tp_scatter_splitk")


def reduce_slots(slots: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Sum over the leading (source-rank) dimension in fp32 (one kernel on CUDA)."""
    n = slots[0].numel()
    if slots.is_cuda and out_dtype == torch.bfloat16 and n % 8 == 0 and slots.stride(0) % 8 == 0 and slots[0].is_contiguous():
        lib = _lib.kernels()
        f = lib.sb_reduce_slots
        if not getattr(f, "_configured", False):
            f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
                          ctypes.c_longlong, ctypes.c_void_p]
            f._configured = True
        out = torch.empty(slots.shape[1:], device=slots.device, dtype=torch.bfloat16)
        _lib.check(f(slots.data_ptr(), slots.shape[0], slots.stride(0), int(slots.dtype == torch.float32), out.data_ptr(), n,
                     _lib.stream_ptr()), "sb_reduce_slots")
        return out
    return slots.float().sum(0).to(out_dtype)


# ----------------------------------------------------------------------------- reference (any backend)
def ref_all_gather_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, 0)


def ref_reduce_scatter_rows(y: torch.Tensor, group=None) -> torch.Tensor:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return y
    W, r = dist.get_world_size(group), dist.get_rank(group)
    y32 = y.float().contiguous()
    dist.all_reduce(y32, group=group)
    per = y.shape[0] // W
    return y32[r * per : (r + 1) * per].to(y.dtype)


class _ColumnParallelFn(torch.autograd.Function):
    """y_local[T, N/tp] = all_gather_rows(x_shard) @ W_shard^T; backward reduce-scatters dx over rows."""

    @staticmethod
    def forward(ctx, x_shard, w, bias, tp: "TPGroup"):
        from ..ops import gemm

        ctx.tp = tp
        R, K = x_shard.shape
        if tp.fused and x_shard.is_cuda:
            buf = tp.gather_buffer(tp.size * R, K, "col_x")
            buf.local.view(tp.size * R, K)[tp.rank * R : (tp.rank + 1) * R].copy_(x_shard)
            tp.peer.barrier()
            y = gemm_all_gather(tp, buf, R, w, bias)
            x_full = buf.local.view(tp.size * R, K).clone()
        else:
            x_full = ref_all_gather_rows(x_shard, tp.group)
            y = gemm.gemm_nt(x_full, w, bias)
        ctx.save_for_backward(x_full, w)
        ctx.has_bias = bias is not None
        ctx.w_main_grad = getattr(w, "main_grad", None)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import gemm

        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        R = x_full.shape[0] // tp.size
        if tp.fused and dy.is_cuda:
            # bf16 slots: the partial tiles cross NVLink at 2 bytes per element (as an NCCL bf16 reduce-scatter would
            # send them) and are added in fp32 by the slot sum
            slots = tp.slot_buffer(R, w.shape[1], torch.bfloat16, "col_dx")
            gemm_reduce_scatter(tp, dy, w, slots, R, w_is_kn=True)
            tp.peer.barrier()
            dx = reduce_slots(slots.local.view(tp.size, R, w.shape[1]), x_full.dtype)
            tp.peer.barrier(1)  # the slots may be overwritten only after every rank has read its own
        else:
            dx = ref_reduce_scatter_rows(gemm.gemm_nn(dy, w), tp.group)
        mg = ctx.w_main_grad
        if mg is not None:
            gemm.gemm_tn(dy, x_full, out=mg.view(w.shape), accumulate=True)
            dw = None
        else:
            dw = gemm.gemm_tn(dy, x_full)
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None


class _RowParallelFn(torch.autograd.Function):
    """y_shard[T/tp, N] = reduce_scatter_rows(x_local[T, K/tp] @ W_shard^T); backward all-gathers dy."""

    @staticmethod
    def forward(ctx, x_local, w, tp: "TPGroup"):
        from ..ops import gemm

        ctx.tp = tp
        T = x_local.shape[0]
        R = T // tp.size
        N = w.shape[0]
        if tp.fused and x_local.is_cuda:
            slots = tp.slot_buffer(R, N, torch.bfloat16, "row_y")
            gemm_reduce_scatter(tp, x_local.contiguous(), w, slots, R)
            tp.peer.barrier()
            y = reduce_slots(slots.local.view(tp.size, R, N), x_local.dtype)
            tp.peer.barrier(1)
        else:
            y = ref_reduce_scatter_rows(gemm.gemm_nt(x_local, w), tp.group)
        ctx.save_for_backward(x_local, w)
        ctx.w_main_grad = getattr(w, "main_grad", None)
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        from ..ops import gemm

        x_local, w = ctx.saved_tensors
        tp = ctx.tp
        R, N = dy_shard.shape
        if tp.fused and dy_shard.is_cuda:
            buf = tp.gather_buffer(tp.size * R, N, "row_dy")
            buf.local.view(tp.size * R, N)[tp.rank * R : (tp.rank + 1) * R].copy_(dy_shard)
            tp.peer.barrier()
            dx = gemm_all_gather(tp, buf, R, w, None, w_is_kn=True)
            dy_full = buf.local.view(tp.size * R, N).clone()
        else:
            dy_full = ref_all_gather_rows(dy_shard.contiguous(), tp.group)
            dx = gemm.gemm_nn(dy_full, w)
        mg = ctx.w_main_grad
        if mg is not None:
            gemm.gemm_tn(dy_full, x_local, out=mg.view(w.shape), accumulate=True)
            dw = None
        else:
            dw = gemm.gemm_tn(dy_full, x_local)
        return dx, dw, None


def column_parallel_linear(x_shard: torch.Tensor, w_shard: torch.Tensor, bias_shard: Optional[torch.Tensor], tp: TPGroup):
    """Sequence-sharded input ``[T/tp, K]`` -> feature-sharded output ``[T, N/tp]``."""
    return _ColumnParallelFn.apply(x_shard, w_shard, bias_shard, tp)


def row_parallel_linear(x_local: torch.Tensor, w_shard: torch.Tensor, tp: TPGroup):
    """Feature-sharded input ``[T, K/tp]`` -> sequence-sharded output ``[T/tp, N]`` (sum over ranks)."""
    return _RowParallelFn.apply(x_local, w_shard, tp)
