"""RMSNorm (optionally fused with the residual add), rotary embedding and SwiGLU.

CUDA tensors run the hand-written kernels in ``csrc/elementwise.cu``; CPU tensors run the PyTorch
reference below (same rounding points: the residual stream is rounded to the activation dtype
before the norm statistics are taken).  These replace the eager HF module code the reference runs
under FSDP (skyrl/backends/skyrl_train/workers/model_wrapper.py:329-333, kernel row K3 of the
device-kernel inventory).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

_cfg_done = False


def _k():
    global _cfg_done
    lib = _lib.kernels()
    if not _cfg_done:
        vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        lib.sb_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, cf, vp]
        lib.sb_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, vp]
        lib.sb_rope_inplace.argtypes = [vp, vp, vp, ci, ci, ci, ci, cf, vp]
        lib.sb_swiglu_fwd.argtypes = [vp, vp, cl, ci, vp]
        lib.sb_swiglu_bwd.argtypes = [vp, vp, vp, cl, ci, vp]
        _cfg_done = True
    return lib


# ----------------------------------------------------------------------------- RMSNorm
def _rmsnorm_ref(x, delta, w, eps):
    if delta is not None:
        x = (x.float() + delta.float()).to(x.dtype)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * w.float()).to(x.dtype)
    return x, y, rstd.squeeze(-1)


class _AddRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, w, eps):
        T, H = x.shape
        if x.is_cuda:
            x = x.contiguous()
            y = torch.empty_like(x)
            rstd = torch.empty(T, device=x.device, dtype=torch.float32)
            if delta is not None:
                delta = delta.contiguous()
                x_out = torch.empty_like(x)
            else:
                x_out = x
            code = _k().sb_rmsnorm_fwd(x.data_ptr(), _lib.ptr(delta), w.data_ptr(),
                                       x_out.data_ptr() if delta is not None else None, y.data_ptr(), rstd.data_ptr(),
                                       T, H, eps, _lib.stream_ptr())
            _lib.check(code, "sb_rmsnorm_fwd")
        else:
            x_out, y, rstd = _rmsnorm_ref(x, delta, w, eps)
        ctx.save_for_backward(x_out, w, rstd)
        # taken here, not from the saved tensor: activation checkpointing hands backward a detached alias of w
        ctx.main_grad = getattr(w, "main_grad", None)
        ctx.has_delta = delta is not None
        ctx.mark_non_differentiable(rstd)
        return x_out, y

    @staticmethod
    def backward(ctx, dx_out, dy):
        x, w, rstd = ctx.saved_tensors
        T, H = x.shape
        main_grad = ctx.main_grad
        if x.is_cuda:
            dy = dy.contiguous()
            dres = dx_out.contiguous() if dx_out is not None else None
            dx = torch.empty_like(x)
            if main_grad is not None:
                dw_buf = main_grad
            else:
                dw_buf = torch.zeros(H, device=x.device, dtype=torch.float32)
            code = _k().sb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres),
                                       dx.data_ptr(), dw_buf.data_ptr(), T, H, _lib.stream_ptr())
            _lib.check(code, "sb_rmsnorm_bwd")
            dw = None if main_grad is not None else dw_buf.to(w.dtype)
        else:
            xf = x.float()
            xhat = xf * rstd[:, None]
            g = dy.float() * w.float()
            dxf = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
            if dx_out is not None:
                dxf = dxf + dx_out.float()
            dx = dxf.to(x.dtype)
            dwf = (dy.float() * xhat).sum(0)
            if main_grad is not None:
                main_grad.add_(dwf)
                dw = None
            else:
                dw = dwf.to(w.dtype)
        return dx, (dx if ctx.has_delta else None), dw, None


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, eps: float):
    """``x_new = x + delta`` (or ``x`` if ``delta`` is None); returns ``(x_new, rmsnorm(x_new) * w)``."""
    return _AddRMSNormFn.apply(x, delta, w, eps)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    shp = x.shape
    _, y = _AddRMSNormFn.apply(x.reshape(-1, shp[-1]), None, w, eps)
    return y.reshape(shp)


# ----------------------------------------------------------------------------- RoPE
def build_rope_table(max_pos: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """[max_pos, head_dim] fp32: cos in the first half of each row, sin in the second."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float().to(device)


def _rope_ref(qkv, pos, table, n_rot_heads, D, sign):
    T = qkv.shape[0]
    half = D // 2
    cs = table[pos.long()]
    cos, sin = cs[:, None, :half], cs[:, None, half:] * sign
    rot = qkv[:, : n_rot_heads * D].reshape(T, n_rot_heads, D).float()
    a, b = rot[..., :half], rot[..., half:]
    out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(qkv.dtype)
    res = qkv.clone()
    res[:, : n_rot_heads * D] = out.reshape(T, n_rot_heads * D)
    return res


def rope_(qkv: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, n_rot_heads: int, head_dim: int,
          sign: float = 1.0) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads of every row of ``qkv`` in place (CUDA) / functionally (CPU)."""
    if qkv.is_cuda:
        assert qkv.stride(1) == 1 and pos.dtype == torch.int32
        code = _k().sb_rope_inplace(qkv.data_ptr(), pos.data_ptr(), table.data_ptr(), qkv.shape[0], n_rot_heads,
                                    qkv.stride(0), head_dim, sign, _lib.stream_ptr())
        _lib.check(code, "sb_rope_inplace")
        return qkv
    return _rope_ref(qkv, pos, table, n_rot_heads, head_dim, sign)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, table, n_rot_heads, head_dim):
        ctx.save_for_backward(pos, table)
        ctx.meta = (n_rot_heads, head_dim)
        if qkv.is_cuda:
            ctx.mark_dirty(qkv)
        return rope_(qkv, pos, table, n_rot_heads, head_dim, 1.0)

    @staticmethod
    def backward(ctx, d):
        pos, table = ctx.saved_tensors
        n, D = ctx.meta
        d = d.contiguous() if d.is_cuda else d
        return rope_(d.clone() if d.is_cuda else d, pos, table, n, D, -1.0), None, None, None, None


def rope(qkv, pos, table, n_rot_heads, head_dim):
    return _RopeFn.apply(qkv, pos, table, n_rot_heads, head_dim)


# ----------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        T, F2 = gu.shape
        F = F2 // 2
        ctx.save_for_backward(gu)
        if gu.is_cuda:
            gu = gu.contiguous()
            out = torch.empty((T, F), device=gu.device, dtype=gu.dtype)
            _lib.check(_k().sb_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, F, _lib.stream_ptr()), "sb_swiglu_fwd")
            return out
        g, u = gu[:, :F].float(), gu[:, F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        T, F2 = gu.shape
        F = F2 // 2
        if gu.is_cuda:
            dout = dout.contiguous()
            dgu = torch.empty_like(gu)
            _lib.check(_k().sb_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, F, _lib.stream_ptr()),
                       "sb_swiglu_bwd")
            return dgu
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), dout.float()
        sig = torch.sigmoid(g)
        silu = g * sig
        return torch.cat([d * u * (sig + silu * (1 - sig)), d * silu], dim=-1).to(gu.dtype)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gu[:, :F]) * gu[:, F:]`` for the fused gate/up projection output."""
    return _SwiGLUFn.apply(gu)


def swiglu_backward(gu: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """Gradient of ``swiglu`` w.r.t. ``gu`` (for hand-written backward passes)."""
    ctx = type("_Ctx", (), {"saved_tensors": (gu,)})()
    return _SwiGLUFn.backward(ctx, dout)


# ----------------------------------------------------------------------------- split-K consumers (decode)
def add_rmsnorm_partials_(x: torch.Tensor, partials: torch.Tensor, n_part: int, w: torch.Tensor, eps: float,
                          out: torch.Tensor | None = None) -> torch.Tensor:
    """``x += sum(partials[:n_part])`` in place (bf16 residual stream), returns ``rmsnorm(x) * w``.

    ``partials`` is the fp32 ``[P, T, H]`` output of ``gemm_nt_splitk``; summing it here saves the separate
    reduction pass a split-K GEMM otherwise needs."""
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        x.copy_((x.float() + partials[:n_part].sum(0)).to(x.dtype))
        out.copy_(_rmsnorm_ref(x, None, w, eps)[1])
        return out
    lib = _lib.kernels()
    f = lib.sb_add_rmsnorm_partials
    if not getattr(f, "_configured", False):
        vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        f.argtypes = [vp, vp, ci, cl, vp, vp, ci, ci, cf, vp]
        f._configured = True
    assert x.is_contiguous() and partials.dtype == torch.float32 and partials.stride(1) == H
    _lib.check(f(x.data_ptr(), partials.data_ptr(), n_part, partials.stride(0), w.data_ptr(), out.data_ptr(), T, H, eps,
                 _lib.stream_ptr()), "sb_add_rmsnorm_partials")
    return out


def qkv_finalize(partials: torch.Tensor, n_part: int, pos: torch.Tensor, table: torch.Tensor, qkv: torch.Tensor,
                 k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, slots: torch.Tensor | None, nq: int,
                 nkv: int, head_dim: int) -> torch.Tensor:
    """Sum the fp32 partials of the fused QKV projection, rotate q/k, write bf16 ``qkv`` and scatter k/v rows
    into their paged-cache slot (one kernel for what was reduction + RoPE + cache write)."""
    T = qkv.shape[0]
    if k_cache is not None:
        _lib.check_index("qkv_finalize: cache slot", slots, k_cache.shape[0] * k_cache.shape[1], min_value=-(1 << 31))
    _lib.check_index("qkv_finalize: position", pos, table.shape[0])
    if not qkv.is_cuda:
        full = partials[:n_part].sum(0).to(qkv.dtype)
        full = _rope_ref(full, pos, table, nq + nkv, head_dim, 1.0)
        qkv.copy_(full)
        if k_cache is not None and slots is not None:
            ok = slots >= 0
            s = slots[ok].long()
            kc = k_cache.view(-1, nkv * head_dim)
            vc = v_cache.view(-1, nkv * head_dim)
            kc[s] = full[ok, nq * head_dim:(nq + nkv) * head_dim]
            vc[s] = full[ok, (nq + nkv) * head_dim:]
        return qkv
    lib = _lib.kernels()
    f = lib.sb_qkv_finalize
    if not getattr(f, "_configured", False):
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        f.argtypes = [vp, ci, cl, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
        f._configured = True
    assert qkv.is_contiguous() and partials.stride(1) == qkv.shape[1] and pos.dtype == torch.int32
    _lib.check(f(partials.data_ptr(), n_part, partials.stride(0), pos.data_ptr(), table.data_ptr(),
                 None if slots is None else slots.data_ptr(), qkv.data_ptr(),
                 None if k_cache is None else k_cache.data_ptr(), None if v_cache is None else v_cache.data_ptr(),
                 T, nq, nkv, head_dim, _lib.stream_ptr()), "sb_qkv_finalize")
    return qkv


# ----------------------------------------------------------------------------- persistent decode block (decode)
class DecodeMlpWorkspace:
    """Buffers of ``decode_mlp_block`` for up to ``max_rows`` sequences: allocated once (outside any CUDA-graph
    capture) and shared by every layer and every batch size, because the kernel uses only a prefix of each."""

    MAX_ROWS = 256

    def __init__(self, max_rows: int, H: int, Q: int, F: int, device, dtype=torch.bfloat16):
        self.max_rows = min(int(max_rows), self.MAX_ROWS)
        self.H, self.Q, self.F = H, Q, F
        lib = _lib.kernels()
        lib.sb_decode_mlp_part_elems.restype = ctypes.c_longlong
        lib.sb_decode_mlp_part_elems.argtypes = [ctypes.c_int] * 4
        elems = int(lib.sb_decode_mlp_part_elems(self.max_rows, H, Q, F))
        self.part = torch.empty(max(elems, 1), device=device, dtype=torch.float32)
        self.h_mid = torch.empty((self.max_rows, H), device=device, dtype=dtype)
        self.act = torch.empty((self.max_rows, F), device=device, dtype=dtype)
        self.h_out = torch.empty((self.max_rows, H), device=device, dtype=dtype)
        self.bar = torch.zeros(1, device=device, dtype=torch.int64)  # arrival counter of the grid barrier
        self.trace = None  # set to an int64 [n_sm, 16] tensor to record per-CTA phase timestamps

    @staticmethod
    def supports(H: int, Q: int, F: int) -> bool:
        return H % 128 == 0 and Q % 64 == 0 and F % 64 == 0 and H // 8 <= 192 * 4


def decode_mlp_block(att: torch.Tensor, x: torch.Tensor, wo: torch.Tensor, ln_mid: torch.Tensor, wgu: torch.Tensor,
                     wd: torch.Tensor, ln_out: torch.Tensor, eps: float, ws: DecodeMlpWorkspace) -> torch.Tensor:
    """Attention output -> next layer's normed input in one persistent kernel (``csrc/decode_mlp.cu``):
    ``x += att @ wo^T``; ``h = rmsnorm(x) * ln_mid``; ``x += (silu(h @ wg^T) * (h @ wu^T)) @ wd^T``; returns
    ``rmsnorm(x) * ln_out`` (a view of the workspace).  ``x`` is updated in place.  What the unfused decode path does
    with five kernels (two split-K GEMMs, the CTA-pair gate/up GEMM and two partial-sum consumers)."""
    n, H = x.shape
    Q, F = att.shape[1], wd.shape[1]
    assert n <= ws.max_rows and (H, Q, F) == (ws.H, ws.Q, ws.F) and x.is_contiguous() and att.is_contiguous()
    lib = _lib.kernels()
    f = lib.sb_decode_mlp_block
    if not getattr(f, "_configured", False):
        vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        f.argtypes = [vp] * 11 + [cl, vp, ci, ci, ci, ci, cf, vp, vp]
        f._configured = True
    out = ws.h_out[:n]
    _lib.check(f(att.data_ptr(), x.data_ptr(), wo.data_ptr(), ln_mid.data_ptr(), wgu.data_ptr(), wd.data_ptr(),
                 ln_out.data_ptr(), ws.h_mid.data_ptr(), ws.act.data_ptr(), out.data_ptr(), ws.part.data_ptr(),
                 ws.part.numel(), ws.bar.data_ptr(), n, H, Q, F, eps, _lib.stream_ptr(), _lib.ptr(ws.trace)),
               "sb_decode_mlp_block")
    return out
