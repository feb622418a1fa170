"""Grouped (per-expert) linear layers for mixture-of-experts FFNs: one kernel launch for all experts.

Rows routed to the same expert are laid out contiguously, each expert's range padded to a multiple of 128 rows, so
that every 128-row tile of the tcgen05 GEMM belongs to exactly one expert.  The plan (row offsets, tile -> expert
table) is computed with device ops and read by the kernel from device memory: no expert count ever reaches the host,
so a layer costs three launches instead of three per expert and can be captured in a CUDA graph.

Reference behaviour: Megatron-core's grouped expert GEMM, enabled with ``moe_grouped_gemm``
(skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:472-473).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

ROW_ALIGN = 128


class GroupPlan:
    """Layout of ``n`` routed rows over ``E`` experts in a padded ``[M_cap, *]`` buffer."""

    def __init__(self, k_off, tile_expert, m_cap, num_experts, top_k, row_src, slot_row, ids, order=None, dst_row=None):
        self.k_off = k_off              # [E + 1] int32 first padded row of each expert (multiples of 128)
        self.tile_expert = tile_expert  # [M_cap / 128] int32 owner of each row block, -1 = unused
        self.m_cap = m_cap
        self.num_experts = num_experts
        self.top_k = top_k
        self.row_src = row_src          # [M_cap] int32 token whose hidden row fills padded row r, -1 = padding
        self.slot_row = slot_row        # [n] int32 padded row of routed entry (token * top_k + slot)
        self._ids, self._order, self._dst_row = ids, order, dst_row

    @property
    def order(self) -> torch.Tensor:
        """[n] routed entries sorted by expert (stable); derived on demand when the plan came from the kernel."""
        if self._order is None:
            self._order = torch.argsort(self._ids.reshape(-1).long(), stable=True)
        return self._order

    @property
    def dst_row(self) -> torch.Tensor:
        """[n] padded-buffer row of sorted entry i."""
        if self._dst_row is None:
            self._dst_row = self.slot_row.long()[self.order]
        return self._dst_row


def padded_rows(n: int, num_experts: int) -> int:
    """Static upper bound of the padded row count for ``n`` routed rows."""
    cap = n + min(num_experts, n) * (ROW_ALIGN - 1)
    return max(ROW_ALIGN, (cap + ROW_ALIGN - 1) // ROW_ALIGN * ROW_ALIGN)


def plan_groups(expert_ids: torch.Tensor, num_experts: int, top_k: int = 1) -> GroupPlan:
    """``expert_ids``: [n] expert of every routed entry; entry ``i`` belongs to token ``i // top_k``.  On CUDA the whole
    plan is one single-CTA kernel (histogram, padded offsets, stable placement); the CPU path spells it out."""
    n = expert_ids.numel()
    dev = expert_ids.device
    m_cap = padded_rows(n, num_experts)
    if expert_ids.is_cuda and num_experts <= 1024 and expert_ids.dtype in (torch.int32, torch.int64):
        ids = expert_ids.reshape(-1).contiguous()
        k_off = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        te = torch.empty(m_cap // ROW_ALIGN, dtype=torch.int32, device=dev)
        row_src = torch.empty(m_cap, dtype=torch.int32, device=dev)
        slot_row = torch.empty(max(n, 1), dtype=torch.int32, device=dev)[:n]
        lib = _lib.kernels()
        if not getattr(lib.sb_moe_plan, "_configured", False):
            vp, ci = ctypes.c_void_p, ctypes.c_int
            lib.sb_moe_plan.restype = ci
            lib.sb_moe_plan.argtypes = [vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp]
            lib.sb_moe_plan._configured = True
        code = lib.sb_moe_plan(ids.data_ptr(), int(ids.dtype == torch.int64), n, num_experts, top_k, m_cap, k_off.data_ptr(),
                               te.data_ptr(), row_src.data_ptr(), slot_row.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sb_moe_plan")
        return GroupPlan(k_off, te, m_cap, num_experts, top_k, row_src, slot_row, ids)
    flat = expert_ids.reshape(-1).long()
    counts = torch.bincount(flat, minlength=num_experts)
    pad = (counts + (ROW_ALIGN - 1)) // ROW_ALIGN * ROW_ALIGN
    ends = torch.cumsum(pad, 0)
    off = ends - pad
    order = torch.argsort(flat, stable=True)
    se = flat[order]
    ustart = torch.cumsum(counts, 0) - counts
    dst_row = off[se] + (torch.arange(n, device=dev) - ustart[se])
    starts = torch.arange(m_cap // ROW_ALIGN, device=dev) * ROW_ALIGN
    te = torch.searchsorted(ends, starts, right=True)
    te = torch.where(starts < ends[-1], te, torch.full_like(te, -1))
    k_off = torch.cat([torch.zeros(1, dtype=ends.dtype, device=dev), ends]).to(torch.int32)
    row_src = torch.full((m_cap,), -1, dtype=torch.int32, device=dev)
    row_src[dst_row] = (order // top_k).to(torch.int32)
    slot_row = torch.empty(n, dtype=torch.int32, device=dev)
    slot_row[order] = dst_row.to(torch.int32)
    return GroupPlan(k_off, te.to(torch.int32), m_cap, num_experts, top_k, row_src, slot_row, flat, order, dst_row)


def _fn():
    lib = _lib.kernels()
    f = lib.sb_gemm_grouped
    if not getattr(f, "_configured", False):
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        f.restype = ci
        f.argtypes = [vp, vp, vp, ci, ci, ci, cl, cl, cl, ci, ci, ci, ci, vp, vp, cl, ci, vp]
        f._configured = True
    return f


def _out_mode(out: torch.Tensor, accumulate: bool) -> int:
    return 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)


def _expert_ranges(plan: GroupPlan):
    k = plan.k_off.tolist()
    return [(e, k[e], k[e + 1]) for e in range(plan.num_experts) if k[e + 1] > k[e]]


def grouped_nt(x: torch.Tensor, w: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """``x`` [M_cap, K] (rows grouped by expert), ``w`` [E, N, K] -> [M_cap, N] with row r times its expert's ``w^T``.
    Rows of unused blocks are left unwritten."""
    M, K = x.shape
    E, N, _ = w.shape
    if not x.is_cuda:
        out = x.new_zeros((M, N))
        for e, lo, hi in _expert_ranges(plan):
            out[lo:hi] = x[lo:hi] @ w[e].t()
        return out
    x, w = x.contiguous(), w.contiguous()
    out = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    code = _fn()(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, 0, 0, 1, E, plan.tile_expert.data_ptr(), None, 0,
                 0, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_grouped(nt)")
    return out


def grouped_nn(dy: torch.Tensor, w: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """``dy`` [M_cap, N], ``w`` [E, N, K] -> [M_cap, K] with row r times its expert's ``w``."""
    M, N = dy.shape
    E, _, K = w.shape
    if not dy.is_cuda:
        out = dy.new_zeros((M, K))
        for e, lo, hi in _expert_ranges(plan):
            out[lo:hi] = dy[lo:hi] @ w[e]
        return out
    dy, w = dy.contiguous(), w.contiguous()
    out = torch.empty((M, K), device=dy.device, dtype=torch.bfloat16)
    # contraction length N (rows of each expert's matrix), output width K
    code = _fn()(dy.data_ptr(), w.data_ptr(), out.data_ptr(), M, K, N, N, K, K, 1, 0, 1, E, plan.tile_expert.data_ptr(), None, 0,
                 0, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_grouped(nn)")
    return out


def grouped_tn(dy: torch.Tensor, x: torch.Tensor, plan: GroupPlan, out: torch.Tensor, accumulate: bool) -> torch.Tensor:
    """``out[e] (+)= dy[rows_e]^T x[rows_e]``; ``dy`` [M_cap, N], ``x`` [M_cap, K], ``out`` [E, N, K].  Padding rows of
    both operands must be zero (or finite in one and zero in the other).  Experts without rows keep ``out[e]``."""
    M, N = dy.shape
    K = x.shape[1]
    E = out.shape[0]
    if not dy.is_cuda:
        for e, lo, hi in _expert_ranges(plan):
            g = dy[lo:hi].float().t() @ x[lo:hi].float()
            if accumulate:
                out[e] += g.to(out.dtype)
            else:
                out[e] = g.to(out.dtype)
        return out
    dy, x = dy.contiguous(), x.contiguous()
    assert out.is_contiguous()
    code = _fn()(dy.data_ptr(), x.data_ptr(), out.data_ptr(), N, K, 0, N, K, K, 1, _out_mode(out, accumulate), 2, E, None,
                 plan.k_off.data_ptr(), N * K, M, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_grouped(tn)")
    return out


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, plan: GroupPlan):
        ctx.plan = plan
        ctx.w_main_grad = getattr(w, "main_grad", None)
        ctx.save_for_backward(x, w)
        return grouped_nt(x, w, plan)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        plan = ctx.plan
        dy = dy.contiguous()
        dx = grouped_nn(dy, w, plan) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = ctx.w_main_grad
            if mg is not None:
                grouped_tn(dy, x, plan, mg.view(w.shape), accumulate=True)
            else:
                dw = grouped_tn(dy, x, plan, torch.zeros_like(w), accumulate=False)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """Differentiable ``x[r] @ w[expert(r)]^T`` over a padded, expert-grouped row buffer.  For the weight gradient the
    padding rows of ``x`` and of the incoming gradient must be zero (``torch.zeros`` + ``index_copy`` gives that)."""
    return _GroupedLinearFn.apply(x, w, plan)


# ----------------------------------------------------------------------------- token movement around the expert GEMMs
def _moe_fns():
    lib = _lib.kernels()
    if not getattr(lib.sb_moe_gather_rows, "_configured", False):
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.sb_moe_gather_rows.argtypes = [vp, vp, vp, ci, ci, vp]
        lib.sb_moe_combine.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp]
        lib.sb_moe_combine_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
        for f in (lib.sb_moe_gather_rows, lib.sb_moe_combine, lib.sb_moe_combine_bwd):
            f.restype = ci
        lib.sb_moe_gather_rows._configured = True
    return lib


def _gather_rows(h: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    if not h.is_cuda:
        out = h.new_zeros((plan.m_cap, h.shape[1]))
        valid = plan.row_src >= 0
        out[valid] = h[plan.row_src[valid].long()]
        return out
    h = h.contiguous()
    out = torch.empty((plan.m_cap, h.shape[1]), device=h.device, dtype=h.dtype)
    code = _moe_fns().sb_moe_gather_rows(h.data_ptr(), plan.row_src.data_ptr(), out.data_ptr(), plan.m_cap, h.shape[1],
                                         _lib.stream_ptr())
    _lib.check(code, "sb_moe_gather_rows")
    return out


def _combine(y: torch.Tensor, plan: GroupPlan, w: torch.Tensor | None, T: int) -> torch.Tensor:
    k, H = plan.top_k, y.shape[1]
    if not y.is_cuda:
        rows = y[plan.slot_row.long()].view(T, k, H).float()
        if w is not None:
            rows = rows * w.float().view(T, k, 1)
        return rows.sum(1).to(y.dtype)
    out = torch.empty((T, H), device=y.device, dtype=y.dtype)
    code = _moe_fns().sb_moe_combine(y.data_ptr(), plan.slot_row.data_ptr(), None if w is None else w.data_ptr(),
                                     out.data_ptr(), T, k, H, _lib.stream_ptr())
    _lib.check(code, "sb_moe_combine")
    return out


def _combine_bwd(y: torch.Tensor | None, plan: GroupPlan, w: torch.Tensor | None, dout: torch.Tensor, want_dw: bool):
    T, H = dout.shape
    k = plan.top_k
    if not dout.is_cuda:
        dy = dout.new_zeros((plan.m_cap, H))
        g = dout.float().view(T, 1, H).expand(T, k, H)
        if w is not None:
            g = g * w.float().view(T, k, 1)
        dy[plan.slot_row.long()] = g.reshape(T * k, H).to(dout.dtype)
        dw = (y[plan.slot_row.long()].view(T, k, H).float() * dout.float().view(T, 1, H)).sum(-1) if want_dw else None
        return dy, dw
    dout = dout.contiguous()
    dy = torch.zeros((plan.m_cap, H), device=dout.device, dtype=dout.dtype)
    dw = torch.empty((T, k), device=dout.device, dtype=torch.float32) if want_dw else None
    code = _moe_fns().sb_moe_combine_bwd(None if y is None else y.data_ptr(), plan.slot_row.data_ptr(),
                                         None if w is None else w.data_ptr(), dout.data_ptr(), dy.data_ptr(),
                                         None if dw is None else dw.data_ptr(), T, k, H, _lib.stream_ptr())
    _lib.check(code, "sb_moe_combine_bwd")
    return dy, dw


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, plan: GroupPlan):
        ctx.plan, ctx.T = plan, h.shape[0]
        return _gather_rows(h, plan)

    @staticmethod
    def backward(ctx, dx):
        return _combine(dx.contiguous(), ctx.plan, None, ctx.T), None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, w, plan: GroupPlan):
        ctx.plan = plan
        w32 = w.float().contiguous()
        ctx.w_dtype = w.dtype
        ctx.save_for_backward(y, w32)
        return _combine(y, plan, w32, w.shape[0])

    @staticmethod
    def backward(ctx, dout):
        y, w32 = ctx.saved_tensors
        dy, dw = _combine_bwd(y, ctx.plan, w32, dout, ctx.needs_input_grad[1])
        return dy, (dw.to(ctx.w_dtype) if dw is not None else None), None


def dispatch_rows(h: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """``[T, H]`` hidden rows -> padded expert-grouped buffer ``[M_cap, H]`` (padding rows zero); the gradient sums
    each token's ``top_k`` rows."""
    return _DispatchFn.apply(h, plan)


def combine_rows(y: torch.Tensor, w: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """``out[t] = sum_s w[t, s] * y[row of (t, s)]`` with ``w`` ``[T, top_k]``; differentiable in ``y`` and ``w``."""
    return _CombineFn.apply(y, w, plan)


def weighted_slot_sum(y_slots: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_s w[t, s] * y_slots[t, s]`` for ``y_slots`` ``[T, k, H]`` (fp32 accumulation, no autograd)."""
    T, k, H = y_slots.shape
    if not y_slots.is_cuda or k > 16 or H % 8 != 0:
        return (y_slots.float() * w.float().unsqueeze(-1)).sum(1).to(y_slots.dtype)
    y = y_slots.contiguous().view(T * k, H)
    rows = torch.arange(T * k, device=y.device, dtype=torch.int32)
    w32 = w.float().contiguous()
    out = torch.empty((T, H), device=y.device, dtype=y.dtype)
    code = _moe_fns().sb_moe_combine(y.data_ptr(), rows.data_ptr(), w32.data_ptr(), out.data_ptr(), T, k, H, _lib.stream_ptr())
    _lib.check(code, "sb_moe_combine")
    return out
