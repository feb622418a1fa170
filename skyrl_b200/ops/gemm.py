"""bf16 GEMMs on the tcgen05 tensor-core kernel (``csrc/gemm_tcgen05.cu``) and the autograd
``linear`` built from them.

The three products of a linear layer map onto one kernel with different operand "major-ness", so
no transposed copy of activations, gradients or weights is ever made:

* ``y  = x  @ W^T``  -> ``gemm_nt``  (A K-major,  B K-major)
* ``dx = dy @ W``    -> ``gemm_nn``  (A K-major,  B MN-major)
* ``dW = dy^T @ x``  -> ``gemm_tn``  (A MN-major, B MN-major), optional fp32 accumulation

CPU tensors take a PyTorch fp32 reference path (used by the CPU test-suite and the gloo plumbing
runs).  Replaces the cuBLAS calls behind ``torch.nn.Linear`` in the reference's HF model forward
(skyrl/backends/skyrl_train/workers/model_wrapper.py:329-333).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_configured = False


def _fn():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        lib.sb_gemm_bf16.restype = ctypes.c_int
        lib.sb_gemm_bf16.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
        ]  # fmt: skip
        _configured = True
    return lib.sb_gemm_bf16


def _as_2d_rowmajor(t: torch.Tensor) -> torch.Tensor:
    assert t.dim() == 2
    if t.stride(1) != 1 or (t.stride(0) % 8) != 0 or (t.data_ptr() % 16) != 0:
        t = t.contiguous()
        if (t.stride(0) % 8) != 0:
            raise ValueError(f"GEMM operand row length {t.shape[1]} must be a multiple of 8")
    return t


def _launch(a, b, c, bias, M, N, K, a_mn, b_mn, out_mode, bn_hint=0):
    code = _fn()(
        a.data_ptr(), b.data_ptr(), c.data_ptr(), None if bias is None else bias.data_ptr(),
        M, N, K, a.stride(0), b.stride(0), c.stride(0), int(a_mn), int(b_mn), out_mode, bn_hint,
        _lib.stream_ptr(),
    )  # fmt: skip
    _lib.check(code, "sb_gemm_bf16")


def gemm_nt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
            out_dtype: torch.dtype | None = None, bn_hint: int = 0, static_w: bool = False) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T (+ bias[N])`` -> ``[M,N]`` (dtype of ``x`` unless ``out_dtype`` is given).
    ``static_w``: ``w`` is not written by any kernel queued before this call (inference weights); its first tiles are
    then fetched while the preceding kernel is still finishing."""
    M, K = x.shape
    N = w.shape[0]
    if out_dtype is None:
        out_dtype = x.dtype
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        y = y.to(out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    x = _as_2d_rowmajor(x)
    w = _as_2d_rowmajor(w)
    if out is None:
        out = torch.empty((M, N), device=x.device, dtype=out_dtype)
    assert out.stride(1) == 1
    mode = 0 if out.dtype == torch.bfloat16 else 1
    _launch(x, w, out, bias, M, N, K, False, False, mode, bn_hint | (0x1000 if static_w else 0))
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, bn_hint: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[K,N]`` -> bf16 ``[M,N]`` (b row-major, i.e. N contiguous)."""
    M, K = a.shape
    N = b.shape[1]
    if not a.is_cuda:
        y = (a.float() @ b.float()).to(a.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    a = _as_2d_rowmajor(a)
    b = _as_2d_rowmajor(b)
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.bfloat16)
    _launch(a, b, out, None, M, N, K, False, True, 0, bn_hint)
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
            out_dtype: torch.dtype | None = None, bn_hint: int = 0) -> torch.Tensor:
    """``a[K,M]^T @ b[K,N]`` -> ``[M,N]``; with ``accumulate`` the fp32 ``out`` is added to."""
    K, M = a.shape
    N = b.shape[1]
    if out_dtype is None:
        out_dtype = a.dtype
    if not a.is_cuda:
        y = a.float().t() @ b.float()
        if out is not None:
            if accumulate:
                out.add_(y.to(out.dtype))
            else:
                out.copy_(y)
            return out
        return y.to(out_dtype)
    a = _as_2d_rowmajor(a)
    b = _as_2d_rowmajor(b)
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    if accumulate:
        assert out.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if out.dtype == torch.bfloat16 else 1
    _launch(a, b, out, None, M, N, K, True, True, mode, bn_hint)
    return out


def plan_splitk(M: int, N: int, K: int, n_sm: int = 148) -> tuple[int, int]:
    """(splits, bn) for a skinny ``x[M,K] @ w[N,K]^T``: enough (tile, k-slice) work items to cover the SMs
    once, with the widest N tile that still does (wide tiles re-read the activation block less often)."""
    m_blocks = (M + 127) // 128
    k_blocks = (K + 63) // 64
    best = (1, 64)
    for bn in (128, 64):
        tiles = m_blocks * ((N + bn - 1) // bn)
        if tiles >= n_sm:
            return 1, bn
        splits = max(1, min(n_sm // tiles, k_blocks // 4 if k_blocks >= 8 else 1))
        best = (splits, bn)
        if tiles * splits >= 0.75 * n_sm:
            break
    splits, bn = best
    if splits > 1:  # no empty slice
        kpb = (k_blocks + splits - 1) // splits
        splits = (k_blocks + kpb - 1) // kpb
    return splits, bn


def gemm_nt_splitk(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, splits: int,
                   bn: int = 64) -> int:
    """``x @ w^T`` as ``splits`` fp32 partial sums written to ``out[s]`` (``out``: fp32 ``[>=splits, M, N]``);
    the bias is folded into partial 0.  Returns the number of partials actually written (<= ``splits``);
    a fused consumer (``add_rmsnorm_partials`` / ``qkv_finalize``) adds them up."""
    M, K = x.shape
    N = w.shape[0]
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        out[0].copy_(y)
        return 1
    lib = _lib.kernels()
    f = lib.sb_gemm_bf16_splitk
    if not getattr(f, "_configured", False):
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                      ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong,
                      ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
        f._configured = True
    assert out.dtype == torch.float32 and out.dim() == 3 and out.shape[0] >= splits and out.stride(2) == 1
    x = _as_2d_rowmajor(x)
    w = _as_2d_rowmajor(w)
    used = ctypes.c_int(0)
    code = f(x.data_ptr(), w.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(), M, N, K,
             x.stride(0), w.stride(0), out.stride(1), out.stride(0), splits, bn, ctypes.byref(used), _lib.stream_ptr())
    _lib.check(code, "sb_gemm_bf16_splitk")
    return used.value


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with all three GEMMs on the tcgen05 kernel.

    If the weight carries a ``main_grad`` fp32 buffer (set by the sharded optimizer) the weight
    gradient is accumulated straight into it by the GEMM epilogue and ``None`` is returned to autograd.
    """

    @staticmethod
    def forward(ctx, x, w, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = gemm_nt(x2, w, bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        # fp32 gradient buffers are looked up on the live parameters now: under activation checkpointing the tensors
        # handed back by ``saved_tensors`` are detached aliases without the attribute
        ctx.w_main_grad = getattr(w, "main_grad", None)
        ctx.b_main_grad = getattr(bias, "main_grad", None) if bias is not None else None
        ctx.in_shape = shp
        return y if x.dim() == 2 else y.reshape(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, w).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main_grad = ctx.w_main_grad
            if main_grad is not None:
                gemm_tn(dy2, x2, out=main_grad, accumulate=True)
            else:
                dw = gemm_tn(dy2, x2, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            bias_main = ctx.b_main_grad
            if bias_main is not None:
                bias_main.add_(dy2.float().sum(0))
            else:
                db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    return _LinearFn.apply(x, w, bias)


def gemm_2cta(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None, a_mn: bool = False,
              b_mn: bool = False, accumulate: bool = False, bn: int = 256) -> torch.Tensor:
    """Low-level entry to the CTA-pair kernel (``csrc/gemm_2cta.cu``): ``out = op(a) op(b) (+ bias)`` with the same
    operand-layout flags as the one-CTA kernel.  ``out`` decides the output mode (bf16 / fp32 / fp32 accumulate)."""
    lib = _lib.kernels()
    f = lib.sb_gemm_bf16_2cta
    if not getattr(f, "_configured", False):
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                      ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                      ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        f._configured = True
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    mode = 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)
    code = f(a.data_ptr(), b.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(), M, N, K, a.stride(0),
             b.stride(0), out.stride(0), int(a_mn), int(b_mn), mode, bn, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_bf16_2cta")
    return out


# ----------------------------------------------------------------------------- fused SwiGLU MLP
def _mlp_fns():
    lib = _lib.kernels()
    f = lib.sb_mlp_gate_up_swiglu
    if not getattr(f, "_configured", False):
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        f.restype = ci
        f.argtypes = [vp, vp, vp, vp, ci, ci, ci, cl, cl, vp]
        lib.sb_mlp_down_dgrad.restype = ci
        lib.sb_mlp_down_dgrad.argtypes = [vp, vp, vp, vp, ci, ci, ci, cl, cl, vp]
        f._configured = True
    return lib


def mlp_fusable(x: torch.Tensor, wgu: torch.Tensor, wd: torch.Tensor) -> bool:
    """The fused epilogues need CUDA bf16 operands, ``F`` a multiple of 128 and enough rows to fill the CTA pairs."""
    F = wd.shape[1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] >= 512 and F % 128 == 0
            and wgu.shape[0] == 2 * F and x.shape[1] % 8 == 0 and os.environ.get("SB_FUSED_MLP", "1") != "0")


def gate_up_swiglu(x: torch.Tensor, wgu: torch.Tensor, need_gu: bool = True):
    """``gu = x @ wgu^T`` and ``act = silu(gu[:, :F]) * gu[:, F:]`` from one GEMM (SwiGLU in the epilogue).  With
    ``need_gu=False`` (forward-only) ``gu`` is neither stored nor returned (``None``)."""
    M, K = x.shape
    F = wgu.shape[0] // 2
    x = _as_2d_rowmajor(x)
    wgu = _as_2d_rowmajor(wgu)
    gu = torch.empty((M, 2 * F), device=x.device, dtype=torch.bfloat16) if need_gu else None
    act = torch.empty((M, F), device=x.device, dtype=torch.bfloat16)
    code = _mlp_fns().sb_mlp_gate_up_swiglu(x.data_ptr(), wgu.data_ptr(), None if gu is None else gu.data_ptr(),
                                            act.data_ptr(), M, F, K, x.stride(0), wgu.stride(0), _lib.stream_ptr())
    _lib.check(code, "sb_mlp_gate_up_swiglu")
    return gu, act


def down_dgrad_swiglu(dy: torch.Tensor, wd: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    """``d(gu)`` of ``swiglu(gu) @ wd^T`` given ``dy``: the product ``dy @ wd`` is consumed in the GEMM epilogue."""
    M, H = dy.shape
    F = wd.shape[1]
    dy = _as_2d_rowmajor(dy)
    wd = _as_2d_rowmajor(wd)
    dgu = torch.empty((M, 2 * F), device=dy.device, dtype=torch.bfloat16)
    code = _mlp_fns().sb_mlp_down_dgrad(dy.data_ptr(), wd.data_ptr(), gu.data_ptr(), dgu.data_ptr(), M, F, H, dy.stride(0),
                                        wd.stride(0), _lib.stream_ptr())
    _lib.check(code, "sb_mlp_down_dgrad")
    return dgu


class _SwiGLUMLPFn(torch.autograd.Function):
    """``swiglu(x Wgu^T) Wd^T`` with the activation fused into the GEMM epilogues in both directions: the forward
    writes ``gu`` and ``act`` from the gate/up GEMM, the backward turns ``dy Wd`` into ``d(gu)`` without storing it."""

    @staticmethod
    def forward(ctx, x, wgu, wd):
        need = any(ctx.needs_input_grad)
        gu, act = gate_up_swiglu(x, wgu, need_gu=need)
        y = gemm_nt(act, wd)
        if need:
            ctx.save_for_backward(x, wgu, wd, gu, act)
        ctx.wgu_main, ctx.wd_main = getattr(wgu, "main_grad", None), getattr(wd, "main_grad", None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wgu, wd, gu, act = ctx.saved_tensors
        dy = dy.contiguous()
        dwd = dwgu = None
        if ctx.wd_main is not None:
            gemm_tn(dy, act, out=ctx.wd_main, accumulate=True)
        else:
            dwd = gemm_tn(dy, act, out_dtype=wd.dtype)
        dgu = down_dgrad_swiglu(dy, wd, gu)
        dx = gemm_nn(dgu, wgu) if ctx.needs_input_grad[0] else None
        if ctx.wgu_main is not None:
            gemm_tn(dgu, x, out=ctx.wgu_main, accumulate=True)
        else:
            dwgu = gemm_tn(dgu, x, out_dtype=wgu.dtype)
        return dx, dwgu, dwd


def swiglu_mlp(x: torch.Tensor, wgu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """Dense SwiGLU feed-forward block.  Large CUDA batches take the fused-epilogue path; everything else is the plain
    composition (``linear`` -> ``swiglu`` -> ``linear``)."""
    if mlp_fusable(x, wgu, wd):
        return _SwiGLUMLPFn.apply(x, wgu, wd)
    from . import elementwise as ew

    return linear(ew.swiglu(linear(x, wgu)), wd)
