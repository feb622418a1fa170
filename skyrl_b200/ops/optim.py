"""Flat fused AdamW and gradient-norm kernels (``csrc/elementwise.cu``).

The optimizer state is three flat fp32 buffers (master weights, first and second moments) per
rank; one launch updates the whole shard and writes the bf16 parameters the model computes
with.  Global-norm clipping never leaves the device: ``sqnorm`` accumulates the squared norm,
``clip_coef`` turns it (after any cross-rank reduction) into a scale factor and a "non-finite, skip"
flag which the AdamW kernel reads.  Semantics follow the reference's optimizer step
(skyrl/backends/skyrl_train/distributed/fsdp_strategy.py:152-186): clip by global norm, skip the step
when the norm is not finite, AdamW with decoupled weight decay.
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
        vp, cf, cl = ctypes.c_void_p, ctypes.c_float, ctypes.c_longlong
        lib.sb_adamw_flat.argtypes = [vp, vp, vp, vp, vp, cl, cf, cf, cf, cf, cf, cf, cf, vp, vp, vp]
        lib.sb_sqnorm_accum.argtypes = [vp, cl, vp, vp]
        lib.sb_clip_coef.argtypes = [vp, cf, cf, vp, vp, vp, vp]
        _cfg_done = True
    return lib


def sqnorm_accum(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out[0] += sum(x**2)`` for a flat fp32 tensor."""
    if x.is_cuda:
        _lib.check(_k().sb_sqnorm_accum(x.data_ptr(), x.numel(), out.data_ptr(), _lib.stream_ptr()), "sb_sqnorm_accum")
    else:
        out[0] += x.float().pow(2).sum()


def clip_coef(sq: torch.Tensor, max_norm: float, extra_scale: float, coef: torch.Tensor, skip: torch.Tensor,
              norm_out: torch.Tensor) -> None:
    """coef = extra_scale * min(1, max_norm / (|extra_scale| * sqrt(sq) + 1e-6)); skip = norm not finite."""
    if sq.is_cuda:
        _lib.check(_k().sb_clip_coef(sq.data_ptr(), max_norm, extra_scale, coef.data_ptr(), skip.data_ptr(),
                                     norm_out.data_ptr(), _lib.stream_ptr()), "sb_clip_coef")
        return
    norm = sq[0].sqrt() * abs(extra_scale)
    finite = bool(torch.isfinite(norm))
    c = extra_scale
    if max_norm > 0 and finite:
        c *= min(1.0, max_norm / (float(norm) + 1e-6))
    coef[0] = c
    skip[0] = 0 if finite else 1
    norm_out[0] = norm


def adamw_flat(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
               param_bf16: torch.Tensor | None, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
               step: int, grad_scale: torch.Tensor | None = None, skip_flag: torch.Tensor | None = None) -> None:
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = master.numel()
    if master.is_cuda:
        code = _k().sb_adamw_flat(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), _lib.ptr(param_bf16),
                                  n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, _lib.ptr(grad_scale),
                                  _lib.ptr(skip_flag), _lib.stream_ptr())
        _lib.check(code, "sb_adamw_flat")
        return
    if skip_flag is not None and int(skip_flag[0]) != 0:
        return
    g = grad.float() * (float(grad_scale[0]) if grad_scale is not None else 1.0)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    master.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if param_bf16 is not None:
        param_bf16.copy_(master)
