"""Small tensor helpers shared by the algorithms and workers."""

from __future__ import annotations

from typing import Optional

import torch


def masked_mean(x: torch.Tensor, mask: Optional[torch.Tensor], dim: Optional[int] = None) -> torch.Tensor:
    """Mean of ``x`` over positions where ``mask`` is non-zero (plain mean if ``mask`` is None)."""
    if mask is None:
        return x.mean() if dim is None else x.mean(dim)
    if dim is None:
        return (x * mask).sum() / mask.sum().clamp(min=1.0)
    return (x * mask).sum(dim) / mask.sum(dim).clamp(min=1.0)


def safe_exp_delta(delta: torch.Tensor, clip: float = 20.0, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``exp(clamp(delta, -clip, clip))`` in fp32, cast back to ``out_dtype``."""
    y = torch.exp(torch.clamp(delta.float(), min=-clip, max=clip))
    return y.to(out_dtype) if out_dtype is not None else y


def masked_var(x: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(x, mask)
    var = masked_mean((x - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("masked_var: the mask selects no element")
        if n == 1:
            raise ValueError("masked_var: the mask selects one element; the unbiased variance is undefined")
        var = var * (n / (n - 1))
    return var


def masked_whiten(x: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mean, var = masked_mean(x, mask), masked_var(x, mask)
    y = (x - mean) * torch.rsqrt(var + 1e-8)
    return y if shift_mean else y + mean


def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor, inplace_backward: bool = False) -> torch.Tensor:
    """Reference-path token log-probabilities from materialised logits (CPU tests and tiny models)."""
    lse = torch.logsumexp(logits.float(), dim=-1)
    return logits.float().gather(-1, labels.unsqueeze(-1)).squeeze(-1) - lse


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lp = torch.log_softmax(logits.float(), dim=-1)
    return -(lp.exp() * lp).sum(-1)


def chunked_entropy_from_logits(logits: torch.Tensor, chunk: int = 1024, attention_mask: Optional[torch.Tensor] = None,
                                requires_grad: bool = False) -> torch.Tensor:
    """Entropy of every position of ``[B, S, V]`` logits, ``chunk`` positions at a time; positions with
    ``attention_mask == 0`` get 0 (reference: utils/torch_utils.py ``chunked_entropy_from_logits``).  The training
    path never calls this -- the fused LM-head kernel yields the entropy without logits -- it is here for code written
    against logits."""
    if attention_mask is not None and tuple(attention_mask.shape) != tuple(logits.shape[:2]):
        raise ValueError(f"attention_mask shape {tuple(attention_mask.shape)} does not match logits shape {tuple(logits.shape[:2])}")
    with torch.set_grad_enabled(requires_grad):
        out = torch.cat([entropy_from_logits(logits[:, i : i + chunk]) for i in range(0, logits.shape[1], chunk)], dim=1)
    return out * attention_mask.to(out.dtype) if attention_mask is not None else out


def chunked_cross_entropy_from_log_probs(logprobs: torch.Tensor, chunk: int = 1024, requires_grad: bool = False) -> torch.Tensor:
    """``-sum_v p_v log p_v`` per position from ``[B, S, V]`` log-probabilities (same role as above)."""
    with torch.set_grad_enabled(requires_grad):
        parts = []
        for i in range(0, logprobs.shape[1], chunk):
            lp = logprobs[:, i : i + chunk].float()
            parts.append(-(lp.exp() * lp).sum(-1))
        return torch.cat(parts, dim=1)
