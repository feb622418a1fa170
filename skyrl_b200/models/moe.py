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
from ..ops import gemm


def route_topk(h: torch.Tensor, router_w: torch.Tensor, top_k: int, norm_topk_prob: bool):
    """Returns (weights [T, k] fp32, expert ids [T, k]); router math in fp32 like the reference config."""
    logits = h.float() @ router_w.float().t()
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
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = torch.arange(T, device=h.device).repeat_interleave(top_k)[order]
    counts = torch.bincount(flat_e, minlength=E).tolist()
    x = h[tok]  # rows grouped by expert
    out_rows = []
    s = 0
    for e in range(E):
        n = counts[e]
        if n == 0:
            continue
        xe = x[s : s + n]
        w1, w2 = wgu[e], wd[e]
        if qat is not None and qat.enabled and torch.is_grad_enabled():  # fake-INT4 expert weights, straight-through
            from .qat import fake_int4

            w1 = fake_int4(w1, qat.group_size, True, qat.scale_divisor, qat.q_min)
            w2 = fake_int4(w2, qat.group_size, True, qat.scale_divisor, qat.q_min)
        gu = gemm.linear(xe, w1)
        out_rows.append(gemm.linear(ew.swiglu(gu), w2))
        s += n
    y = torch.cat(out_rows, dim=0) if out_rows else x.new_zeros((0, H))
    wf = w.reshape(-1)[order].to(y.dtype)
    out = torch.zeros((T, H), device=h.device, dtype=torch.float32)
    out.index_add_(0, tok, (y * wf[:, None]).float())
    return out.to(h.dtype)
