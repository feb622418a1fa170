"""Ulysses sequence parallelism: tokens are sharded over the ``sp`` ranks everywhere except inside attention, where
heads are sharded instead; the two all-to-alls that switch layouts are fused into the projections around attention.

Reference: skyrl/backends/skyrl_train/distributed/ulysses/{utils,monkey_patch}.py (three ``all_to_all`` calls on q, k, v
before flash-attention and one after, plus an all-gather of position ids; utils.py:138-167, monkey_patch.py:53-124).
Here:

* ``qkv_proj``: the QKV GEMM's epilogue stores every 32-column chunk straight into the memory of the rank that owns
  those heads (one kernel instead of GEMM + 3 all-to-alls); positions / cu_seqlens are known on every rank already.
* ``o_proj``: copy warps inside the output projection pull the other ranks' head blocks for this rank's tokens while
  the tensor cores start on the blocks that have landed (one kernel instead of all-to-all + GEMM).
* backward passes and CPU / gloo runs use ``all_to_all_single`` (``seq_to_head`` / ``head_to_seq``).

``sp`` must divide both the query and the key/value head counts (the reference replicates KV heads when ``sp`` exceeds
them; that case is rejected here).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib, gemm
from .tensor_parallel import TPGroup

_cfg = False


def _k():
    global _cfg
    lib = _lib.kernels()
    if not _cfg:
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.sb_gemm_sp.argtypes = [vp, vp, vp, vp, ci, ci, ci, cl, cl, cl, ci, vp, ci, ci, ci, vp, vp, ci, cl, vp, ci, vp]
        _cfg = True
    return lib


def _segments(widths: Sequence[int], sp: int) -> Tuple[list, list]:
    """Column segments (q | k | v) of the fused projection -> (start of each, width per rank)."""
    starts, per, off = [], [], 0
    for w in widths:
        if w % sp:
            raise ValueError(f"segment width {w} does not divide by sp={sp}")
        starts.append(off)
        per.append(w // sp)
        off += w
    while len(starts) < 3:
        starts.append(off)
        per.append(0)
    return starts, per


def seq_to_head(x: torch.Tensor, widths: Sequence[int], sp: TPGroup) -> torch.Tensor:
    """``[R, sum(widths)]`` (my tokens, all heads) -> ``[sp*R, sum(widths)/sp]`` (all tokens, my heads)."""
    if sp.size == 1:
        return x
    R = x.shape[0]
    starts, per = _segments(widths, sp.size)
    send = torch.cat([torch.cat([x[:, s + d * p : s + (d + 1) * p] for s, p in zip(starts, per) if p], 1)
                      for d in range(sp.size)], 0).contiguous()  # [sp*R, local]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=sp.group)
    return recv


def head_to_seq(x: torch.Tensor, widths: Sequence[int], sp: TPGroup) -> torch.Tensor:
    """Inverse of ``seq_to_head``."""
    if sp.size == 1:
        return x
    R = x.shape[0] // sp.size
    starts, per = _segments(widths, sp.size)
    recv = torch.empty_like(x)
    dist.all_to_all_single(recv, x.contiguous(), group=sp.group)  # block s = rank s's heads for my tokens
    out = torch.empty((R, sum(widths)), dtype=x.dtype, device=x.device)
    for srank in range(sp.size):
        blk = recv[srank * R : (srank + 1) * R]
        o = 0
        for s, p in zip(starts, per):
            if p:
                out[:, s + srank * p : s + (srank + 1) * p] = blk[:, o : o + p]
                o += p
    return out


class _QKVProjFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, bias, widths, sp: TPGroup):
        ctx.sp, ctx.widths, ctx.has_bias = sp, tuple(widths), bias is not None
        ctx.w_main_grad = getattr(w, "main_grad", None)
        ctx.save_for_backward(h, w)
        R, K = h.shape
        N = w.shape[0]
        if sp.fused and h.is_cuda and R % 1 == 0:
            starts, per = _segments(widths, sp.size)
            local = sum(per)
            buf = sp.slot_buffer(R, local, torch.bfloat16, "ulysses_qkv")  # [sp, R, local] == [sp*R, local]
            sp.peer.barrier(2)  # every rank has finished reading the previous contents
            outs = (ctypes.c_void_p * sp.size)(*buf.ptrs)
            ss = (ctypes.c_int * 3)(*starts)
            sw = (ctypes.c_int * 3)(*per)
            code = _k().sb_gemm_sp(h.data_ptr(), w.data_ptr(), None, None if bias is None else bias.data_ptr(), R, N, K,
                                   h.stride(0), w.stride(0), local, 1, outs, sp.size, sp.rank, R, ss, sw, 0, 0, None, 0,
                                   _lib.stream_ptr())
            _lib.check(code, "sb_gemm_sp(scatter)")
            sp.peer.barrier()
            return buf.local.view(sp.size * R, local).clone()
        return seq_to_head(gemm.gemm_nt(h, w, bias), widths, sp)

    @staticmethod
    def backward(ctx, dqkv_local):
        h, w = ctx.saved_tensors
        dqkv = head_to_seq(dqkv_local.contiguous(), ctx.widths, ctx.sp)  # [R, N]
        dh = gemm.gemm_nn(dqkv, w)
        mg = ctx.w_main_grad
        if mg is not None:
            gemm.gemm_tn(dqkv, h, out=mg.view(w.shape), accumulate=True)
            dw = None
        else:
            dw = gemm.gemm_tn(dqkv, h)
        db = dqkv.float().sum(0).to(dqkv.dtype) if ctx.has_bias else None
        return dh, dw, db, None, None


class _OProjFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, att_local, w, sp: TPGroup):
        ctx.sp = sp
        ctx.w_main_grad = getattr(w, "main_grad", None)
        T, cpr = att_local.shape
        R = T // sp.size
        H, K = w.shape
        if sp.fused and att_local.is_cuda:
            src = sp.gather_buffer(T, cpr, "ulysses_att")
            sp.peer.barrier(2)
            src.local.view(T, cpr).copy_(att_local)
            sp.peer.barrier()
            a_full = torch.empty((R, K), device=att_local.device, dtype=torch.bfloat16)
            out = torch.empty((R, H), device=att_local.device, dtype=torch.bfloat16)
            peers = (ctypes.c_void_p * sp.size)(*src.ptrs)
            flags = sp.flags((R + 127) // 128)
            code = _k().sb_gemm_sp(a_full.data_ptr(), w.data_ptr(), out.data_ptr(), None, R, H, K, K, w.stride(0), H, 2, peers,
                                   sp.size, sp.rank, R, None, None, cpr, cpr, flags.data_ptr(), 0, _lib.stream_ptr())
            _lib.check(code, "sb_gemm_sp(gather)")
            att_seq = a_full
        else:
            att_seq = head_to_seq(att_local, [K], sp)
            out = gemm.gemm_nt(att_seq, w)
        ctx.save_for_backward(att_seq, w)
        return out

    @staticmethod
    def backward(ctx, dout):
        att_seq, w = ctx.saved_tensors
        dout = dout.contiguous()
        datt_seq = gemm.gemm_nn(dout, w)  # [R, K]
        mg = ctx.w_main_grad
        if mg is not None:
            gemm.gemm_tn(dout, att_seq, out=mg.view(w.shape), accumulate=True)
            dw = None
        else:
            dw = gemm.gemm_tn(dout, att_seq)
        return seq_to_head(datt_seq, [w.shape[1]], ctx.sp), dw, None


def qkv_proj(h_shard: torch.Tensor, wqkv: torch.Tensor, bias: Optional[torch.Tensor], widths: Sequence[int], sp: TPGroup):
    """``[R, H]`` -> ``[sp*R, (q + k + v widths) / sp]``: fused QKV projection + sequence-to-head exchange."""
    return _QKVProjFn.apply(h_shard, wqkv, bias, tuple(widths), sp)


def o_proj(att_local: torch.Tensor, wo: torch.Tensor, sp: TPGroup):
    """``[sp*R, q_width / sp]`` -> ``[R, H]``: head-to-sequence exchange + output projection."""
    return _OProjFn.apply(att_local, wo, sp)
