"""Corrections for the gap between the rollout engine's policy and the trainer's "old" policy.

Truncated importance sampling (token or sequence level), sequence rejection masks (geometric mean
or product of the token ratios), outlier-token sequence rejection and per-token hard masks.
Behavioural reference: skyrl/backends/skyrl_train/utils/off_policy_correction_utils.py:24-385.
Here every correction is one small function of the shared token ratio ``pi_old / pi_rollout`` and
``compute_off_policy_correction`` folds them in a fixed order (outlier mask, token mask, TIS,
sequence mask), each acting on the mask left by the previous one.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..utils.torch_utils import masked_mean, safe_exp_delta


def _flags(cfg):
    tis = cfg.tis_ratio_type is not None
    seq = cfg.sequence_mask_metric is not None
    outlier = cfg.outlier_token_is_threshold_low is not None or cfg.outlier_token_is_threshold_high is not None
    token = cfg.token_mask_is_threshold_low is not None and cfg.token_mask_is_threshold_high is not None
    return tis, seq, outlier, token


def off_policy_correction_enabled(cfg) -> bool:
    return any(_flags(cfg))


def _frac(count: torch.Tensor, total) -> float:
    return (count / total).detach().item()


def compute_tis_ratio(old_log_probs, rollout_logprobs, loss_mask, tis_ratio_type: str, cfg) -> Tuple[torch.Tensor, Dict]:
    log_r = old_log_probs - rollout_logprobs
    if tis_ratio_type == "token":
        r = safe_exp_delta(log_r, 20.0, old_log_probs.dtype)
        cap = cfg.token_tis_ratio_clip_high
        capped = ((r > cap) & (loss_mask > 0)).sum()
        return r.clamp(max=cap).detach(), {"tis_token_clip_high_ratio": _frac(capped, (loss_mask > 0).sum().clamp(min=1))}
    if tis_ratio_type == "sequence":
        r = safe_exp_delta((log_r * loss_mask).sum(-1, keepdim=True), 20.0, old_log_probs.dtype)
        cap = cfg.sequence_tis_ratio_clip_high
        return r.clamp(max=cap).detach(), {"tis_seq_clip_high_ratio": _frac((r > cap).sum(), r.shape[0])}
    raise ValueError(f"Unknown tis_ratio_type: {tis_ratio_type}")


def compute_outlier_token_mask(old_log_probs, rollout_logprobs, loss_mask, cfg) -> Tuple[torch.Tensor, Dict]:
    """Reject whole sequences that contain any token whose ratio leaves ``[low, high]``."""
    r = safe_exp_delta(old_log_probs - rollout_logprobs, 20.0, old_log_probs.dtype)
    live = loss_mask > 0
    zeros = torch.zeros_like(loss_mask, dtype=torch.bool)
    over = (r > cfg.outlier_token_is_threshold_high) & live if cfg.outlier_token_is_threshold_high is not None else zeros
    under = (r < cfg.outlier_token_is_threshold_low) & live if cfg.outlier_token_is_threshold_low is not None else zeros
    keep = (~(over | under) | ~live).all(dim=-1, keepdim=True)
    n = float(keep.shape[0])
    metrics = {
        "outlier_seq_masked_ratio": _frac((~keep.squeeze(-1)).sum(), n),
        "outlier_seq_over_high_ratio": _frac(over.any(-1).sum(), n),
        "outlier_seq_under_low_ratio": _frac(under.any(-1).sum(), n),
    }
    return keep.float(), metrics


def compute_token_mask(old_log_probs, rollout_logprobs, loss_mask, cfg) -> Tuple[torch.Tensor, Dict]:
    """Zero individual tokens whose ratio leaves ``[low, high]``; padded positions stay untouched."""
    r = safe_exp_delta(old_log_probs - rollout_logprobs, 20.0, old_log_probs.dtype)
    inside = (r >= cfg.token_mask_is_threshold_low) & (r <= cfg.token_mask_is_threshold_high)
    live = loss_mask > 0
    metrics = {"token_mask_ratio": _frac((~inside & live).sum(), live.sum().clamp(min=1))}
    return (inside | ~live).float(), metrics


def compute_sequence_mask(old_log_probs, rollout_logprobs, loss_mask, metric: str, cfg) -> Tuple[torch.Tensor, Dict]:
    log_sum = ((old_log_probs - rollout_logprobs) * loss_mask).sum(-1, keepdim=True)
    if metric == "geometric":
        stat = safe_exp_delta(log_sum / loss_mask.sum(-1, keepdim=True).clamp(min=1.0), 20.0, old_log_probs.dtype)
        hi, lo, tag = cfg.geo_mask_high, cfg.geo_mask_low, "geo_sequence_mask"
    elif metric == "product":
        stat = safe_exp_delta(log_sum, 20.0, old_log_probs.dtype)
        hi, lo, tag = cfg.product_mask_high, cfg.product_mask_low, "product_sequence_mask"
    else:
        raise ValueError(f"Unknown sequence_mask_metric: {metric}")
    over, under = stat > hi, stat < lo
    keep = ~over & ~under
    n = float(stat.shape[0])
    metrics = {f"{tag}_masked_ratio": _frac((~keep).sum(), n), f"{tag}_over_high_ratio": _frac(over.sum(), n),
               f"{tag}_under_low_ratio": _frac(under.sum(), n)}
    return keep.float(), metrics


def compute_off_policy_correction(old_log_probs, rollout_logprobs, loss_mask, cfg):
    """Returns ``(tis_ratio or None, metrics, loss_mask')``."""
    tis, seq, outlier, token = _flags(cfg)
    if not (tis or seq or outlier or token):
        return None, {}, loss_mask
    r = safe_exp_delta(old_log_probs - rollout_logprobs, 20.0, old_log_probs.dtype)
    masked = r * loss_mask
    metrics = {"is_ratio_mean": masked_mean(r, loss_mask).mean().item(), "is_ratio_std": masked.std().item(),
               "is_ratio_max": masked.max().item(), "is_ratio_min": masked.min().item()}
    if outlier:
        m, extra = compute_outlier_token_mask(old_log_probs, rollout_logprobs, loss_mask, cfg)
        loss_mask = loss_mask * m
        metrics.update(extra)
    if token:
        m, extra = compute_token_mask(old_log_probs, rollout_logprobs, loss_mask, cfg)
        loss_mask = loss_mask * m
        metrics.update(extra)
    ratio = None
    if tis:
        ratio, extra = compute_tis_ratio(old_log_probs, rollout_logprobs, loss_mask, cfg.tis_ratio_type, cfg)
        metrics.update(extra)
    if seq:
        m, extra = compute_sequence_mask(old_log_probs, rollout_logprobs, loss_mask, cfg.sequence_mask_metric, cfg)
        loss_mask = loss_mask * m
        metrics.update(extra)
    return ratio, metrics, loss_mask


def apply_off_policy_correction(loss, old_log_probs, rollout_logprobs: Optional[torch.Tensor], loss_mask, cfg):
    """Multiply ``loss`` by the TIS ratio and shrink ``loss_mask``; a no-op without rollout log-probs."""
    if rollout_logprobs is None:
        return loss, loss_mask, {}
    ratio, metrics, loss_mask = compute_off_policy_correction(old_log_probs, rollout_logprobs, loss_mask, cfg)
    if ratio is not None:
        loss = loss * ratio
    return loss, loss_mask, metrics
