"""LM-head log-probability and entropy without materialising ``[T, V]`` logits.

Forward is the fused tcgen05 kernel of ``csrc/lmhead_logprob.cu`` (GEMM main loop with an online
softmax epilogue, vocabulary splits merged by a combine kernel).  Backward recomputes the logits of
a bounded block of rows with the plain GEMM, turns them into ``dlogits`` in place with one
elementwise kernel and feeds the two gradient GEMMs, so peak memory is ``rows_per_block * V`` bf16
regardless of sequence length.

With ``tp_group`` the vocabulary is sharded across ranks: each rank reduces its own slice and the
combine step merges the per-rank partial records (max, sum-exp, sum-exp*z, target logit), which is the
whole cross-rank traffic -- 16 bytes per token per split instead of three all-reduces over
``[T]``-sized tensors.  Replaces the reference's ``logprobs_from_logits`` on materialised logits
(skyrl/backends/skyrl_train/utils/torch_utils.py:115-177), its chunked entropy (:58-111) and the
vendored Triton fused LM-head (distributed/megatron/fused_linear_logprob_triton.py).
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib, gemm

_cfg_done = False


def _k():
    global _cfg_done
    lib = _lib.kernels()
    if not _cfg_done:
        vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        lib.sb_lmhead_num_splits.argtypes = [ci, ci]
        lib.sb_lmhead_partials.argtypes = [vp, vp, vp, vp, ci, ci, ci, cl, cl, ci, cf, vp]
        lib.sb_lmhead_combine.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp]
        lib.sb_lmhead_dlogits.argtypes = [vp, cl, ci, ci, vp, ci, vp, vp, vp, vp, cf, vp]
        _cfg_done = True
    return lib


BWD_ROWS_PER_BLOCK = 8192


def _ref_forward(hidden, W, targets, inv_temp, with_entropy, vocab_offset=0):
    z = (hidden.float() @ W.float().t()) * inv_temp
    lse = torch.logsumexp(z, dim=-1)
    lp = z.gather(-1, (targets.long() - vocab_offset).clamp(0, z.shape[1] - 1)[:, None]).squeeze(-1) - lse
    ent = None
    if with_entropy:
        p = torch.softmax(z, dim=-1)
        ent = lse - (p * z).sum(-1)
    return lp, ent, lse


def lm_head_partials(hidden: torch.Tensor, W: torch.Tensor, targets: torch.Tensor, inv_temp: float,
                     vocab_offset: int = 0, out: Optional[torch.Tensor] = None):
    """Per-(row, split) softmax partial records ``[T, splits, 4]`` for this rank's vocabulary slice."""
    T, K = hidden.shape
    V = W.shape[0]
    splits = int(_k().sb_lmhead_num_splits(T, V))
    if callable(out):
        out = out(T, splits)  # e.g. a view into symmetric memory that the peers can read
    if out is None:
        out = torch.empty((T, splits, 4), device=hidden.device, dtype=torch.float32)
    code = _k().sb_lmhead_partials(hidden.data_ptr(), W.data_ptr(), targets.data_ptr(), out.data_ptr(), T, V, K,
                                   hidden.stride(0), W.stride(0), vocab_offset, inv_temp, _lib.stream_ptr())
    _lib.check(code, "sb_lmhead_partials")
    return out, splits


def lm_head_combine(partial_ptrs, splits: int, T: int, device, want_entropy: bool = True):
    n = len(partial_ptrs)
    arr = (ctypes.c_void_p * n)(*partial_ptrs)
    lp = torch.empty(T, device=device, dtype=torch.float32)
    ent = torch.empty(T, device=device, dtype=torch.float32) if want_entropy else None
    lse = torch.empty(T, device=device, dtype=torch.float32)
    code = _k().sb_lmhead_combine(arr, n, splits, T, lp.data_ptr(), _lib.ptr(ent), lse.data_ptr(), _lib.stream_ptr())
    _lib.check(code, "sb_lmhead_combine")
    return lp, ent, lse


class _LMHeadLogprobFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, W, targets, inv_temp, with_entropy, vocab_offset, peer_exchange):
        T = hidden.shape[0]
        if hidden.is_cuda:
            hidden = hidden.contiguous()
            t32 = targets.to(torch.int32).contiguous()
            partials, splits = lm_head_partials(hidden, W, t32, inv_temp, vocab_offset,
                                                out=getattr(peer_exchange, "alloc", None))
            if peer_exchange is not None:
                ptrs = peer_exchange(partials, splits)  # pointers to every rank's records, own included
            else:
                ptrs = [partials.data_ptr()]
            lp, ent, lse = lm_head_combine(ptrs, splits, T, hidden.device, True)
            if peer_exchange is not None and hasattr(peer_exchange, "release"):
                peer_exchange.release()
        else:
            t32 = targets.to(torch.int32)
            lp, ent, lse = _ref_forward(hidden, W, targets, inv_temp, True, vocab_offset)
        ctx.save_for_backward(hidden, W, t32, lse, ent)
        ctx.main_grad = getattr(W, "main_grad", None)  # see ops/gemm.py: not recoverable from the saved alias
        ctx.inv_temp = inv_temp
        ctx.vocab_offset = vocab_offset
        ctx.with_entropy = with_entropy
        if with_entropy:
            return lp, ent
        ctx.mark_non_differentiable(ent)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, W, targets, lse, ent = ctx.saved_tensors
        inv_temp, voff = ctx.inv_temp, ctx.vocab_offset
        T, K = hidden.shape
        V = W.shape[0]
        use_ent = ctx.with_entropy and g_ent is not None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        main_grad = ctx.main_grad
        if not hidden.is_cuda:
            with torch.enable_grad():
                h = hidden.detach().float().requires_grad_()
                w = W.detach().float().requires_grad_()
                lp, e, _ = _ref_forward(h, w, targets, inv_temp, True, voff)
                tot = (lp * g_lp.float()).sum()
                if use_ent:
                    tot = tot + (e * g_ent.float()).sum()
                dh, dw = torch.autograd.grad(tot, (h, w))
            if main_grad is not None:
                main_grad.add_(dw)
                dw = None
            else:
                dw = dw.to(W.dtype)
            return dh.to(hidden.dtype), dw, None, None, None, None, None
        g_lp = g_lp.float().contiguous()
        g_ent_c = g_ent.float().contiguous() if use_ent else None
        dh = torch.empty_like(hidden) if need_dh else None
        dw_acc = None
        if need_dw:
            dw_acc = main_grad if main_grad is not None else torch.zeros((V, K), device=W.device, dtype=torch.float32)
        rows = min(BWD_ROWS_PER_BLOCK, T)
        buf = torch.empty((rows, V), device=hidden.device, dtype=torch.bfloat16)
        for s in range(0, T, rows):
            e = min(T, s + rows)
            n = e - s
            z = buf[:n]
            gemm.gemm_nt(hidden[s:e], W, out=z)
            code = _k().sb_lmhead_dlogits(z.data_ptr(), z.stride(0), n, V, targets[s:e].data_ptr(), voff,
                                          lse[s:e].data_ptr(), ent[s:e].data_ptr() if use_ent else None,
                                          g_lp[s:e].data_ptr(), g_ent_c[s:e].data_ptr() if use_ent else None, inv_temp,
                                          _lib.stream_ptr())
            _lib.check(code, "sb_lmhead_dlogits")
            if need_dh:
                gemm.gemm_nn(z, W, out=dh[s:e])
            if need_dw:
                gemm.gemm_tn(z, hidden[s:e], out=dw_acc, accumulate=True)
        dw = None
        if need_dw and main_grad is None:
            dw = dw_acc.to(W.dtype)
        return dh, dw, None, None, None, None, None


def lm_head_logprobs(hidden: torch.Tensor, W: torch.Tensor, targets: torch.Tensor, inv_temp: float = 1.0,
                     with_entropy: bool = False, vocab_offset: int = 0, peer_exchange=None):
    """Returns ``(logprob [T], entropy [T])`` of ``targets`` under ``softmax(hidden @ W^T * inv_temp)``.

    ``entropy`` is always computed (it is free in the fused epilogue) but only carries a gradient when
    ``with_entropy`` is set.  For vocabulary-parallel use pass this rank's ``vocab_offset`` and a
    ``peer_exchange`` callable that publishes the local partial records and returns the device pointers
    of every rank's records.
    """
    if peer_exchange is None and vocab_offset == 0:  # vocabulary-parallel shards legitimately see foreign targets
        _lib.check_index("lm_head_logprobs: target id", targets, W.shape[0])
    return _LMHeadLogprobFn.apply(hidden, W, targets, inv_temp, with_entropy, vocab_offset, peer_exchange)
