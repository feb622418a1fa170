"""Fake INT4 quantisation-aware training for expert weights: group-wise symmetric quantise -> dequantise in the
forward pass, straight-through gradients (reference: skyrl/backends/skyrl_train/workers/megatron/fake_int4_qat.py:50-146,
groups of 32 along the input dimension, applied to MoE expert GEMM weights)."""

from __future__ import annotations

import torch


def fake_int4_quant_dequant(w: torch.Tensor, group_size: int = 32, scale_divisor: float = 7.0, q_min: float = -7.0,
                            q_max: float = 7.0) -> torch.Tensor:
    """Round ``w`` to 4-bit symmetric levels (``q_min..q_max`` times a per-group scale ``amax / scale_divisor``) along
    the last dimension.  The reference's defaults are ``scale_divisor=7.5, q_min=-8`` (config ``fake_int4_qat``)."""
    shp = w.shape
    K = shp[-1]
    if K % group_size != 0:
        raise ValueError(f"last dimension {K} is not a multiple of the group size {group_size}")
    g = w.float().reshape(-1, K // group_size, group_size)
    scale = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / scale_divisor
    q = torch.clamp(torch.round(g / scale), q_min, q_max)
    return (q * scale).reshape(shp).to(w.dtype)


class _FakeInt4STE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, group_size, scale_divisor, q_min):
        return fake_int4_quant_dequant(w, group_size, scale_divisor, q_min)

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None  # straight-through


def fake_int4(w: torch.Tensor, group_size: int = 32, enabled: bool = True, scale_divisor: float = 7.0,
              q_min: float = -7.0) -> torch.Tensor:
    return _FakeInt4STE.apply(w, group_size, scale_divisor, q_min) if enabled else w


def quantization_error(w: torch.Tensor, group_size: int = 32) -> float:
    return float((fake_int4_quant_dequant(w, group_size).float() - w.float()).norm() / w.float().norm().clamp_min(1e-12))
