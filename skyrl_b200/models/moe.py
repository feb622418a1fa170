"""Mixture-of-experts FFN (Qwen3-MoE style: softmax router, top-k, optional renormalisation).

Tokens are sorted by expert so that each expert's rows are contiguous and every expert runs the
same three tcgen05 GEMM products as a dense FFN on its slice; the expert-parallel variant (dispatch
and combine over peer memory) lives in ``skyrl_b200.parallel.expert_parallel``.  Reference: the
Megatron MoE layer configured at skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:377-545
(``moe_token_dispatcher_type="alltoall"``, ``moe_grouped_gemm``).
"""

from __future__ import annotations

import torch

from ..ops import elementwise as ew
from ..ops import gemm  # noqa: F401
from ..ops import grouped_gemm as gg


class _RouteFn(torch.autograd.Function):
    """softmax -> top-k -> (re)normalise in one kernel per direction (``csrc/moe.cu``)."""

    @staticmethod
    def forward(ctx, logits, top_k, norm):
        import ctypes

        from ..ops import _lib

        lib = _lib.kernels()
        if not getattr(lib.sb_moe_route, "_configured", False):
            vp, ci = ctypes.c_void_p, ctypes.c_int
            lib.sb_moe_route.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
            lib.sb_moe_route_bwd.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
            lib.sb_moe_route.restype = lib.sb_moe_route_bwd.restype = ci
            lib.sb_moe_route._configured = True
        T, E = logits.shape
        logits = logits.contiguous()
        w = torch.empty((T, top_k), device=logits.device, dtype=torch.float32)
        idx = torch.empty((T, top_k), device=logits.device, dtype=torch.int32)
        _lib.check(lib.sb_moe_route(logits.data_ptr(), w.data_ptr(), idx.data_ptr(), T, E, top_k, int(norm), _lib.stream_ptr()),
                   "sb_moe_route")
        ctx.save_for_backward(logits, w, idx)
        ctx.norm, ctx.lib = bool(norm), lib
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, dw, _didx):
        from ..ops import _lib

        logits, w, idx = ctx.saved_tensors
        T, E = logits.shape
        dlogits = torch.empty_like(logits)
        dw = dw.float().contiguous()
        _lib.check(ctx.lib.sb_moe_route_bwd(logits.data_ptr(), w.data_ptr(), idx.data_ptr(), dw.data_ptr(), dlogits.data_ptr(),
                                            T, E, idx.shape[1], int(ctx.norm), _lib.stream_ptr()), "sb_moe_route_bwd")
        return dlogits, None, None


def route_topk(h: torch.Tensor, router_w: torch.Tensor, top_k: int, norm_topk_prob: bool):
    """Returns (weights [T, k] fp32, expert ids [T, k]); router math in fp32 like the reference config."""
    logits = h.float() @ router_w.float().t()
    if logits.is_cuda and logits.shape[1] <= 1024 and top_k <= 16:
        w, idx = _RouteFn.apply(logits, top_k, norm_topk_prob)
        return w, idx.long()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, idx


def moe_ffn(h: torch.Tensor, router_w: torch.Tensor, wgu: torch.Tensor, wd: torch.Tensor, top_k: int,
            norm_topk_prob: bool = True, routed_indices: torch.Tensor | None = None, layer: int | None = None, qat=None) -> torch.Tensor:
    """``h``: [T, H]; ``wgu``: [E, 2F, H]; ``wd``: [E, H, F].  ``routed_indices`` replays rollout-time routing;
    with ``layer`` given, an active ``router_replay`` context records or overrides the choice."""
    T, H = h.shape
    E = wgu.shape[0]
    w, idx = route_topk(h, router_w, top_k, norm_topk_prob)
    if layer is not None and routed_indices is None:
        from . import router_replay

        routed_indices = router_replay.on_route(layer, idx)
    if routed_indices is not None:
        probs = torch.softmax(h.float() @ router_w.float().t(), dim=-1)
        idx = routed_indices.long()
        w = probs.gather(-1, idx)
        if norm_topk_prob:
            w = w / w.sum(dim=-1, keepdim=True)
    plan = gg.plan_groups(idx.reshape(-1), E, top_k)
    # rows grouped by expert, every expert's range padded to whole 128-row tiles (padding rows are zero)
    x = gg.dispatch_rows(h, plan)
    w1, w2 = wgu, wd
    if qat is not None and qat.enabled and torch.is_grad_enabled():  # fake-INT4 expert weights, straight-through
        from .qat import fake_int4

        w1 = fake_int4(w1, qat.group_size, True, qat.scale_divisor, qat.q_min)
        w2 = fake_int4(w2, qat.group_size, True, qat.scale_divisor, qat.q_min)
        # the fp32 gradient buffers belong to the parameters, not to the quantised copies
        for q, prm in ((w1, wgu), (w2, wd)):
            mg = getattr(prm, "main_grad", None)
            if mg is not None:
                q.main_grad = mg
    gu = gg.grouped_linear(x, w1, plan)
    y = gg.grouped_linear(ew.swiglu(gu), w2, plan)
    return gg.combine_rows(y, w, plan)
