"""Expert parallelism for MoE layers: experts are sharded over the ``ep`` ranks, tokens stay data-parallel, and the
two token exchanges (dispatch to the experts' ranks, combine back) run *inside* the expert GEMM kernels.

Reference behaviour: Megatron-core's ``alltoall`` token dispatcher plus grouped expert GEMMs
(skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:472-473, config.py:464-469: ``expert_model_parallel_size``,
``moe_token_dispatcher_type="alltoall"``, ``moe_grouped_gemm``): permute -> all-to-all -> expert MLP -> all-to-all ->
un-permute.  Here, per local expert:

* gate/up GEMM in *dispatch* mode: copy warps fetch each routed token's hidden row straight from the rank that holds
  it (peer loads, indexed by a small routing table) while the tensor cores work on rows that have landed;
* down GEMM in *combine* mode: the epilogue stores each output row into slot ``(token, k)`` of the source rank's
  combine buffer (peer stores); the source then takes the routing-weighted sum over its ``k`` slots.

Only the routing tables (``T x k`` integers per rank) travel through a regular collective.  The backward pass mirrors
the forward with the two modes swapped.  Without CUDA peers (CPU / gloo) the same interface runs an
``all_to_all``-free reference that gathers every rank's tokens, for testing the layer logic.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib, elementwise as ew, gemm
from .tensor_parallel import TPGroup

_cfg = False


def _k():
    global _cfg
    lib = _lib.kernels()
    if not _cfg:
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.sb_gemm_ep.argtypes = [vp, vp, vp, ci, ci, ci, cl, cl, cl, ci, ci, vp, ci, ci, vp, vp, cl, vp, ci, vp]
        lib.sb_gemm_ep_grouped.argtypes = [vp, vp, vp, ci, ci, ci, cl, cl, cl, ci, ci, vp, ci, ci, vp, vp, cl, vp, ci, ci, vp, vp]
        _cfg = True
    return lib


def build_routing_tables(idx: torch.Tensor, ep: TPGroup, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, List[int]]:
    """From this rank's expert choices ``idx [T, k]`` build, for the experts that live on this rank, the rows they must
    process: ``(src_rank [n], src_row [n], dst_row [n], counts per local expert)``, grouped by expert.  ``src_row`` is the
    token's index in its owner's hidden buffer, ``dst_row = token * k + slot`` in the owner's combine buffer."""
    T, k = idx.shape
    E_local = num_experts // ep.size
    if ep.size > 1:
        allidx = [torch.empty_like(idx) for _ in range(ep.size)]
        dist.all_gather(allidx, idx.contiguous(), group=ep.group)
        full = torch.stack(allidx, 0)  # [ep, T, k]  (every rank processes the same number of tokens per micro-batch)
    else:
        full = idx.unsqueeze(0)
    mine = (full // E_local) == ep.rank
    r, t, s = torch.nonzero(mine, as_tuple=True)
    e = full[r, t, s] - ep.rank * E_local
    order = torch.argsort(e, stable=True)
    r, t, s, e = r[order], t[order], s[order], e[order]
    counts = _Counts(torch.bincount(e, minlength=E_local).tolist())
    counts.expert_of_row = e  # [n] local expert of every row (sorted), for the grouped launch
    return r.to(torch.int32).contiguous(), t.to(torch.int32).contiguous(), (t * k + s).to(torch.int32).contiguous(), counts


class _Counts(list):
    """Per-local-expert row counts; also carries the per-row expert ids as an attribute."""

    expert_of_row: Optional[torch.Tensor] = None


class _ExpertParallelFFN(torch.autograd.Function):
    """out[t] = sum_k w[t,k] * FFN_{idx[t,k]}(h[t]) with experts sharded over ``ep``."""

    @staticmethod
    def forward(ctx, h, w, idx, wgu, wd, ep: TPGroup, num_experts: int):
        T, H = h.shape
        k = idx.shape[1]
        E_local, F2 = wgu.shape[0], wgu.shape[1]
        src_rank, src_row, dst_row, counts = build_routing_tables(idx, ep, num_experts)
        n = int(src_rank.numel())
        fused = ep.fused and h.is_cuda
        if fused:
            hbuf = ep.gather_buffer(T, H, "ep_hidden")  # this rank's tokens, readable by peers
            comb = ep.slot_buffer(T * k, H, torch.bfloat16, "ep_combine")  # [ep(unused dim folded), ...]
            ep.peer.barrier(2)  # peers finished reading the previous micro-batch's buffers
            hbuf.local.view(T, H).copy_(h)
            ep.peer.barrier()
            peers_h = (ctypes.c_void_p * ep.size)(*hbuf.ptrs)
            peers_c = (ctypes.c_void_p * ep.size)(*comb.ptrs)
            # one grouped launch per projection: rows padded so that every 128-row tile belongs to one expert
            from ..ops import grouped_gemm as gg

            plan = gg.plan_groups(counts.expert_of_row, E_local)
            Mc = plan.m_cap
            pad_rank = torch.full((Mc,), -1, dtype=torch.int32, device=h.device)
            pad_srow = torch.zeros((Mc,), dtype=torch.int32, device=h.device)
            pad_drow = torch.zeros((Mc,), dtype=torch.int32, device=h.device)
            rows_of = plan.slot_row.long()  # the tables are sorted by expert already: entry i sits in padded row slot_row[i]
            pad_rank[rows_of] = src_rank
            pad_srow[rows_of] = src_row
            pad_drow[rows_of] = dst_row
            ctx.rows_of = rows_of
            x_rows = torch.empty((Mc, H), device=h.device, dtype=h.dtype)
            gu = torch.empty((Mc, F2), device=h.device, dtype=h.dtype)
            flags = ep.flags(Mc // 128 + 2)
            wgu_c, wd_c = wgu.contiguous(), wd.contiguous()
            code = _k().sb_gemm_ep_grouped(x_rows.data_ptr(), wgu_c.data_ptr(), gu.data_ptr(), Mc, F2, H, H, H, F2, 0, 1,
                                           peers_h, ep.size, ep.rank, pad_rank.data_ptr(), pad_srow.data_ptr(), H,
                                           flags.data_ptr(), 256, E_local, plan.tile_expert.data_ptr(), _lib.stream_ptr())
            _lib.check(code, "sb_gemm_ep_grouped(dispatch)")
            act = ew.swiglu(gu)
            code = _k().sb_gemm_ep_grouped(act.data_ptr(), wd_c.data_ptr(), None, Mc, H, F2 // 2, F2 // 2, F2 // 2, H, 0, 2,
                                           peers_c, ep.size, ep.rank, pad_rank.data_ptr(), pad_drow.data_ptr(), 0, None,
                                           256, E_local, plan.tile_expert.data_ptr(), _lib.stream_ptr())
            _lib.check(code, "sb_gemm_ep_grouped(combine)")
            ctx.plan = plan
            ep.peer.barrier()
            y_slots = comb.local[: T * k * H].view(T, k, H).clone()
        else:
            x_rows, gu, act, y_rows = _reference_expert_rows(h, wgu, wd, ep, src_rank, src_row, counts)
            y_slots = _reference_combine(y_rows, ep, src_rank, dst_row, T, k, H)
        from ..ops.grouped_gemm import weighted_slot_sum

        out = weighted_slot_sum(y_slots, w)
        ctx.ep, ctx.num_experts, ctx.counts, ctx.fused = ep, num_experts, counts, fused
        if fused:
            ctx.save_for_backward(w, x_rows, gu, act, y_slots, wgu, wd, src_rank, src_row, dst_row)
        else:
            ctx.plan = None
            ctx.save_for_backward(w, x_rows[:n] if n else x_rows[:0], gu[:n] if n else gu[:0], act, y_slots, wgu, wd,
                                  src_rank, src_row, dst_row)
        ctx.wgu_main, ctx.wd_main = getattr(wgu, "main_grad", None), getattr(wd, "main_grad", None)
        ctx.shape = (T, H, k)
        return out

    @staticmethod
    def backward(ctx, dout):
        w, x_rows, gu, act, y_slots, wgu, wd, src_rank, src_row, dst_row = ctx.saved_tensors
        ep, counts = ctx.ep, ctx.counts
        T, H, k = ctx.shape
        E_local, F2 = wgu.shape[0], wgu.shape[1]
        F = F2 // 2
        n = int(src_rank.numel())
        dout = dout.contiguous()
        dw = (y_slots.float() * dout.float().unsqueeze(1)).sum(-1).to(w.dtype)  # [T, k]
        dy_slots = (dout.float().unsqueeze(1) * w.float().unsqueeze(-1)).to(dout.dtype).reshape(T * k, H).contiguous()
        # "dispatch" the slot gradients to the experts (rows indexed by dst_row on the owner), then mirror the forward
        dy_rows = _exchange_rows_to_experts(dy_slots, ep, src_rank, dst_row, n, H, ctx.fused, "ep_dy")
        dwd = ctx.wd_main if ctx.wd_main is not None else torch.zeros(wd.shape, device=wd.device, dtype=torch.float32)
        dwgu = ctx.wgu_main if ctx.wgu_main is not None else torch.zeros(wgu.shape, device=wgu.device, dtype=torch.float32)
        if ctx.plan is not None:
            # grouped launches over the padded layout saved by the forward pass (padding rows are zero)
            from ..ops import grouped_gemm as gg

            plan = ctx.plan
            dy_pad = torch.zeros((plan.m_cap, H), device=dout.device, dtype=dout.dtype).index_copy(0, ctx.rows_of, dy_rows)
            dact = gg.grouped_nn(dy_pad, wd, plan)
            gg.grouped_tn(dy_pad, act, plan, dwd.view(wd.shape), accumulate=True)
            dgu = ew.swiglu_backward(gu, dact)
            dx_pad = gg.grouped_nn(dgu, wgu, plan)
            gg.grouped_tn(dgu, x_rows, plan, dwgu.view(wgu.shape), accumulate=True)
            dx_rows = dx_pad[ctx.rows_of]
            dh_slots = _fused_combine_rows(dx_rows, ep, src_rank, dst_row, T, k, H)
            dh = dh_slots.float().sum(1).to(dout.dtype)
            return (dh, dw, None, None if ctx.wgu_main is not None else dwgu.to(wgu.dtype),
                    None if ctx.wd_main is not None else dwd.to(wd.dtype), None, None)
        dact = torch.empty((max(n, 1), F), device=dout.device, dtype=dout.dtype)[:n]
        s = 0
        for e in range(E_local):
            c = counts[e]
            if c == 0:
                continue
            dact[s : s + c] = gemm.gemm_nn(dy_rows[s : s + c], wd[e])
            gemm.gemm_tn(dy_rows[s : s + c], act[s : s + c], out=dwd[e], accumulate=True)
            s += c
        dgu = ew.swiglu_backward(gu, dact) if n else gu
        dx_rows = torch.empty((max(n, 1), H), device=dout.device, dtype=dout.dtype)[:n]
        s = 0
        for e in range(E_local):
            c = counts[e]
            if c == 0:
                continue
            dx_rows[s : s + c] = gemm.gemm_nn(dgu[s : s + c], wgu[e])
            gemm.gemm_tn(dgu[s : s + c], x_rows[s : s + c], out=dwgu[e], accumulate=True)
            s += c
        if ctx.fused:
            dh_slots = _fused_combine_rows(dx_rows, ep, src_rank, dst_row, T, k, H)
        else:
            dh_slots = _reference_combine(dx_rows, ep, src_rank, dst_row, T, k, H)
        dh = dh_slots.float().sum(1).to(dout.dtype)
        return (dh, dw, None, None if ctx.wgu_main is not None else dwgu.to(wgu.dtype),
                None if ctx.wd_main is not None else dwd.to(wd.dtype), None, None)


# ----------------------------------------------------------------------------- helpers (reference + exchanges)
def _all_gather_rows(x: torch.Tensor, ep: TPGroup) -> torch.Tensor:
    if ep.size == 1:
        return x.unsqueeze(0)
    parts = [torch.empty_like(x) for _ in range(ep.size)]
    dist.all_gather(parts, x.contiguous(), group=ep.group)
    return torch.stack(parts, 0)


def _reference_expert_rows(h, wgu, wd, ep, src_rank, src_row, counts):
    allh = _all_gather_rows(h, ep)  # [ep, T, H]
    x_rows = allh[src_rank.long(), src_row.long()]
    n = x_rows.shape[0]
    gu = torch.empty((n, wgu.shape[1]), device=h.device, dtype=h.dtype)
    s = 0
    for e, c in enumerate(counts):
        if c:
            gu[s : s + c] = gemm.gemm_nt(x_rows[s : s + c], wgu[e])
            s += c
    act = ew.swiglu(gu) if n else gu.new_zeros((0, wgu.shape[1] // 2))
    y = torch.empty((n, h.shape[1]), device=h.device, dtype=h.dtype)
    s = 0
    for e, c in enumerate(counts):
        if c:
            y[s : s + c] = gemm.gemm_nt(act[s : s + c], wd[e])
            s += c
    return x_rows, gu, act, y


def _reference_combine(y_rows, ep, src_rank, dst_row, T, k, H):
    """Send every row back to (src_rank, dst_row): all-gather the rows and tables, keep what is addressed to me."""
    if ep.size == 1:
        out = torch.zeros((T * k, H), device=y_rows.device, dtype=y_rows.dtype)
        out[dst_row.long()] = y_rows
        return out.view(T, k, H)
    n_local = torch.tensor([y_rows.shape[0]], device=y_rows.device)
    ns = [torch.zeros_like(n_local) for _ in range(ep.size)]
    dist.all_gather(ns, n_local, group=ep.group)
    nmax = int(max(int(x) for x in ns))
    pad = lambda t, fill=0: torch.cat([t, t.new_full((nmax - t.shape[0], *t.shape[1:]), fill)], 0)  # noqa: E731
    rows = _all_gather_rows(pad(y_rows), ep)
    ranks = _all_gather_rows(pad(src_rank, -1), ep)
    drows = _all_gather_rows(pad(dst_row), ep)
    out = torch.zeros((T * k, H), device=y_rows.device, dtype=y_rows.dtype)
    sel = ranks == ep.rank
    out[drows[sel].long()] = rows[sel]
    return out.view(T, k, H)


def _fused_combine_rows(rows, ep, src_rank, dst_row, T, k, H):
    """Row exchange back to the owners through peer stores (identity 'GEMM'-free path: plain indexed push)."""
    comb = ep.slot_buffer(T * k, H, torch.bfloat16, "ep_combine_bwd")
    ep.peer.barrier(2)
    _push_rows(rows, comb, ep, src_rank, dst_row)
    ep.peer.barrier()
    return comb.local[: T * k * H].view(T, k, H).clone()


def _push_rows(rows, comb, ep, dst_rank, dst_row):
    """Store ``rows[i]`` into ``comb`` of rank ``dst_rank[i]`` at row ``dst_row[i]`` (per destination rank, through the
    peer mapping of that rank's buffer)."""
    H = rows.shape[1]
    for d in range(ep.size):
        sel = (dst_rank == d).nonzero(as_tuple=True)[0]
        if sel.numel() == 0:
            continue
        from .peer import _CudaArray

        view = torch.as_tensor(_CudaArray(comb.ptrs[d], comb.local.numel() * 2), device=rows.device).view(torch.bfloat16)
        view.view(-1, H).index_copy_(0, dst_row[sel].long(), rows[sel])


def _exchange_rows_to_experts(slots, ep, src_rank, dst_row, n, H, fused, tag):
    """Fetch, for each expert row, row ``dst_row`` of ``slots`` on rank ``src_rank`` (the backward's dispatch)."""
    if not fused:
        alls = _all_gather_rows(slots, ep)
        return alls[src_rank.long(), dst_row.long()]
    buf = ep.gather_buffer(slots.shape[0], H, tag)
    ep.peer.barrier(2)
    buf.local.view(-1, H).copy_(slots)
    ep.peer.barrier()
    out = torch.empty((n, H), device=slots.device, dtype=slots.dtype)
    from .peer import _CudaArray

    for r in range(ep.size):
        sel = (src_rank == r).nonzero(as_tuple=True)[0]
        if sel.numel():
            view = torch.as_tensor(_CudaArray(buf.ptrs[r], buf.local.numel() * 2), device=slots.device).view(torch.bfloat16)
            out[sel] = view.view(-1, H)[dst_row[sel].long()]
    return out


def moe_ffn_ep(h: torch.Tensor, router_w: torch.Tensor, wgu_local: torch.Tensor, wd_local: torch.Tensor, top_k: int,
               norm_topk_prob: bool, ep: TPGroup, num_experts: int, layer: Optional[int] = None) -> torch.Tensor:
    """Expert-parallel MoE FFN: ``wgu_local`` / ``wd_local`` hold this rank's ``num_experts / ep`` experts."""
    from ..models.moe import route_topk
    from ..models import router_replay

    w, idx = route_topk(h, router_w, top_k, norm_topk_prob)
    forced = router_replay.on_route(layer, idx) if layer is not None else None
    if forced is not None:
        probs = torch.softmax(h.float() @ router_w.float().t(), dim=-1)
        idx = forced.long()
        w = probs.gather(-1, idx)
        if norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
    return _ExpertParallelFFN.apply(h, w, idx, wgu_local, wd_local, ep, num_experts)
