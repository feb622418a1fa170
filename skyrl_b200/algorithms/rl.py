"""RL mathematics: advantage estimators, policy / critic losses, KL estimators and controllers,
loss-reduction pre-scaling, and the registries that let users plug in their own.

Behavioural reference: skyrl/backends/skyrl_train/utils/ppo_utils.py (estimators :1224-1428, losses
:555-1142, KL :88-126, controllers :45-85, reductions :1152-1220, registries :178-403).  The
implementation differs: group statistics are vectorised with ``index_add_`` instead of Python
dictionaries, registries are plain in-process tables (there is no actor to sync with because
workers are spawned after registration and inherit them), and on CUDA the common GRPO + clipped
objective path runs in the fused kernels of ``csrc/rl_loss.cu``.
"""

from __future__ import annotations

import ctypes
from enum import Enum
from typing import Callable, Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from ..ops import _lib
from ..utils.torch_utils import masked_mean, masked_whiten, safe_exp_delta
from .off_policy import apply_off_policy_correction


# ----------------------------------------------------------------------------- registries
class FunctionRegistry:
    """Name -> callable table. Subclasses hold independent tables."""

    _kind = "function"
    _table: Dict[str, Callable]

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        cls._table = {}

    @classmethod
    def register(cls, name: Union[str, Enum], fn: Callable) -> None:
        key = name.value if isinstance(name, Enum) else str(name)
        if key in cls._table and cls._table[key] is not fn:
            raise ValueError(f"{cls._kind} '{key}' already registered")
        cls._table[key] = fn

    @classmethod
    def get(cls, name: Union[str, Enum]) -> Callable:
        key = name.value if isinstance(name, Enum) else str(name)
        if key not in cls._table:
            raise ValueError(f"unknown {cls._kind} '{key}'; available: {sorted(cls._table)}")
        return cls._table[key]

    @classmethod
    def list_available(cls) -> List[str]:
        return sorted(cls._table)

    @classmethod
    def unregister(cls, name: Union[str, Enum]) -> None:
        key = name.value if isinstance(name, Enum) else str(name)
        if key not in cls._table:
            raise ValueError(f"{cls._kind} '{key}' is not registered")
        del cls._table[key]


class AdvantageEstimatorRegistry(FunctionRegistry):
    _kind = "advantage estimator"


class PolicyLossRegistry(FunctionRegistry):
    _kind = "policy loss"


class AdvantageEstimator(str, Enum):
    GAE = "gae"
    GRPO = "grpo"
    RLOO = "rloo"
    REINFORCE_PP = "reinforce++"
    MAXRL = "maxrl"


class PolicyLossType(str, Enum):
    REGULAR = "regular"
    DUAL_CLIP = "dual_clip"
    GSPO = "gspo"
    CISPO = "cispo"
    ROLLOUT_IS = "rollout_is"
    CLIP_COV = "clip_cov"
    KL_COV = "kl_cov"
    SAPO = "sapo"
    CROSS_ENTROPY = "cross_entropy"
    IMPORTANCE_SAMPLING = "importance_sampling"
    DPPO = "dppo"


# losses anchored on the rollout log-probabilities: the "old policy" forward pass can be skipped
LOSSES_WITHOUT_OLD_LOGPROBS = frozenset({"rollout_is", "dppo"})


def register_advantage_estimator(name):
    def deco(fn):
        AdvantageEstimatorRegistry.register(name, fn)
        return fn

    return deco


def register_policy_loss(name):
    def deco(fn):
        PolicyLossRegistry.register(name, fn)
        return fn

    return deco


# ----------------------------------------------------------------------------- KL
class AdaptiveKLController:
    """Proportional controller of https://arxiv.org/abs/1909.08593."""

    def __init__(self, init_kl_coef: float, target: float, horizon: int):
        self.value, self.target, self.horizon = init_kl_coef, target, horizon

    def update(self, current: float, n_steps: int) -> None:
        err = float(np.clip(current / self.target - 1, -0.2, 0.2))
        self.value *= 1 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current: float, n_steps: int) -> None:
        return None


def get_kl_controller(algorithm_cfg):
    kind = algorithm_cfg.kl_ctrl.type
    if kind == "fixed":
        return FixedKLController(algorithm_cfg.kl_loss_coef)
    if kind == "adaptive":
        if algorithm_cfg.kl_ctrl.horizon <= 0:
            raise ValueError(f"horizon must be larger than 0. Got {algorithm_cfg.kl_ctrl.horizon}")
        return AdaptiveKLController(algorithm_cfg.kl_loss_coef, algorithm_cfg.kl_ctrl.kl_target,
                                    algorithm_cfg.kl_ctrl.horizon)
    raise ValueError(f"Invalid KL controller type: {kind}")


def compute_approx_kl(log_probs: torch.Tensor, log_probs_base: torch.Tensor, loss_mask: Optional[torch.Tensor] = None,
                      kl_estimator_type: str = "k3") -> torch.Tensor:
    """Per-token KL estimate (http://joschu.net/blog/kl-approx.html): ``k1``, ``abs``, ``k2`` or ``k3``."""
    d = log_probs - log_probs_base
    if kl_estimator_type == "k1":
        kld = d
    elif kl_estimator_type == "abs":
        kld = d.abs()
    elif kl_estimator_type == "k2":
        kld = 0.5 * d.square()
    elif kl_estimator_type == "k3":
        neg = torch.clamp(-d, min=-20, max=20)
        kld = torch.clamp(torch.exp(neg) - neg - 1, min=-10, max=10)
    else:
        raise ValueError(f"Invalid KL estimator type: {kl_estimator_type}")
    if loss_mask is not None:
        kld = torch.where(loss_mask.bool(), kld * loss_mask, torch.zeros_like(kld))
    return kld


# ----------------------------------------------------------------------------- advantage estimators
def _dense_groups(index) -> Tuple[torch.Tensor, int]:
    """Map arbitrary hashable group labels to dense ids 0..G-1 (first-seen order)."""
    seen: Dict[object, int] = {}
    ids = [seen.setdefault(k if not isinstance(k, np.generic) else k.item(), len(seen)) for k in list(index)]
    return torch.tensor(ids, dtype=torch.long), len(seen)


def _group_stats(scores: torch.Tensor, gid: torch.Tensor, G: int):
    """Per-sample (count, mean, unbiased std) of its group; singleton groups get mean 0 / std 1."""
    s = scores.float()
    gid = gid.to(s.device)
    cnt = torch.zeros(G, device=s.device).index_add_(0, gid, torch.ones_like(s))
    tot = torch.zeros(G, device=s.device).index_add_(0, gid, s)
    mean = torch.where(cnt > 1, tot / cnt.clamp(min=1), torch.zeros_like(tot))
    dev = (s - mean[gid]) ** 2
    ss = torch.zeros(G, device=s.device).index_add_(0, gid, dev)
    std = torch.where(cnt > 1, torch.sqrt(ss / (cnt - 1).clamp(min=1)), torch.ones_like(ss))
    return cnt[gid], mean[gid], std[gid]


_GROUP_MODES = {"grpo": 0, "dr_grpo": 1, "rloo": 2}


def _group_advantage_cuda(scores: torch.Tensor, gid: torch.Tensor, G: int, mode: int, eps: float) -> torch.Tensor:
    lib = _lib.kernels()
    lib.sb_group_advantage.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    s = scores.float().contiguous()
    g32 = gid.to(device=s.device, dtype=torch.int32)
    out = torch.zeros_like(s)
    _lib.check(lib.sb_group_advantage(s.data_ptr(), g32.data_ptr(), s.numel(), G, mode, eps, out.data_ptr(),
                                      _lib.stream_ptr()), "sb_group_advantage")
    return out


@register_advantage_estimator(AdvantageEstimator.GRPO)
def compute_grpo_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index,
                                   epsilon: float = 1e-6, grpo_norm_by_std: bool = True, **kwargs):
    """``(score - mean_group) / (std_group + eps)`` broadcast over the response (Dr.GRPO without the std)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = _dense_groups(index)
        if scores.is_cuda:
            adv = _group_advantage_cuda(scores, gid, G, 0 if grpo_norm_by_std else 1, epsilon).to(scores.dtype)
        else:
            _, mean, std = _group_stats(scores, gid, G)
            adv = (scores - mean) / (std + epsilon) if grpo_norm_by_std else scores - mean
            adv = adv.to(scores.dtype)
        out = adv.unsqueeze(-1) * response_mask
    return out, out


@register_advantage_estimator(AdvantageEstimator.RLOO)
def compute_rloo_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index, **kwargs):
    """Leave-one-out baseline (https://arxiv.org/abs/2402.14740); a lone sample gets advantage 0."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = _dense_groups(index)
        cnt, mean, _ = _group_stats(scores, gid, G)
        adv = torch.where(cnt > 1, (scores - mean) * cnt / (cnt - 1).clamp(min=1), torch.zeros_like(scores))
        out = adv.to(scores.dtype).unsqueeze(-1) * response_mask
    return out, out


@register_advantage_estimator(AdvantageEstimator.MAXRL)
def compute_maxrl_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index,
                            epsilon: float = 1e-6, **kwargs):
    """Mean-normalised group-relative reward ``(s - mean_g) / (mean_g + eps)``."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = _dense_groups(index)
        cnt, mean, _ = _group_stats(scores, gid, G)
        adv = torch.where(cnt > 1, (scores - mean) / (mean + epsilon), scores - mean)
        out = adv.to(scores.dtype).unsqueeze(-1) * response_mask
    return out, out


@register_advantage_estimator(AdvantageEstimator.REINFORCE_PP)
def compute_reinforce_plus_plus_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor,
                                                  gamma: float, **kwargs):
    """REINFORCE++ (https://arxiv.org/abs/2501.03262): discounted return-to-go, reset after EOS, whitened."""
    with torch.no_grad():
        R = token_level_rewards.shape[1]
        returns = torch.zeros_like(token_level_rewards)
        run = torch.zeros_like(token_level_rewards[:, 0])
        for t in range(R - 1, -1, -1):
            run = token_level_rewards[:, t] + gamma * run
            returns[:, t] = run
            run = run * response_mask[:, t]
        adv = masked_whiten(returns, response_mask) * response_mask
    return adv, returns


def _gae_scan(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lambd: float):
    if rewards.is_cuda:
        lib = _lib.kernels()
        lib.sb_gae.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        r, v = rewards.float().contiguous(), values.float().contiguous()
        adv, ret = torch.empty_like(r), torch.empty_like(r)
        _lib.check(lib.sb_gae(r.data_ptr(), v.data_ptr(), None, r.shape[0], r.shape[1], gamma, lambd, adv.data_ptr(),
                              ret.data_ptr(), _lib.stream_ptr()), "sb_gae")
        return adv.to(rewards.dtype), ret.to(rewards.dtype)
    R = rewards.shape[-1]
    adv = torch.zeros_like(rewards)
    last = torch.zeros_like(rewards[:, 0])
    for t in range(R - 1, -1, -1):
        nxt = values[:, t + 1] if t < R - 1 else torch.zeros_like(last)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lambd * last
        adv[:, t] = last
    return adv, adv + values


@register_advantage_estimator(AdvantageEstimator.GAE)
def compute_gae_advantage_return(token_level_rewards: torch.Tensor, values: torch.Tensor, response_mask: torch.Tensor,
                                 gamma: float, lambd: float, **kwargs):
    """Generalised advantage estimation; returns = advantages + values; advantages masked-whitened."""
    with torch.no_grad():
        adv, returns = _gae_scan(token_level_rewards, values, gamma, lambd)
        adv = masked_whiten(adv, response_mask)
    return adv, returns


def compute_advantages_and_returns(token_level_rewards, response_mask, index, adv_estimator, config=None, values=None,
                                   grpo_norm_by_std: bool = True, gamma: float = 1.0, lambd: float = 1.0, **kwargs):
    fn = AdvantageEstimatorRegistry.get(adv_estimator)
    return fn(token_level_rewards=token_level_rewards, response_mask=response_mask, index=index, values=values,
              grpo_norm_by_std=grpo_norm_by_std, gamma=gamma, lambd=lambd, config=config, **kwargs)


# ----------------------------------------------------------------------------- loss reduction
def reduce_loss(loss: torch.Tensor, loss_mask: Optional[torch.Tensor]) -> torch.Tensor:
    return (loss * loss_mask).sum() if loss_mask is not None else loss.sum()


def apply_loss_reduction_to_advantages_minibatch(advantages: torch.Tensor, loss_mask: torch.Tensor,
                                                 loss_reduction: str, micro_batch_size: int, max_seq_len: int,
                                                 prompt_boundaries: Optional[List[Tuple[int, int]]] = None):
    """Scale advantages so that a plain masked *sum* of the token losses realises ``loss_reduction``."""
    B = advantages.shape[0]
    if loss_reduction == "token_mean":
        return advantages / loss_mask.sum().clamp(min=1)
    if loss_reduction == "sequence_mean":
        return advantages / (B * loss_mask.sum(dim=-1, keepdim=True).clamp(min=1))
    if loss_reduction == "seq_mean_token_sum_norm":
        return advantages / (B * max_seq_len)
    out = torch.zeros_like(advantages)
    if loss_reduction == "token_mean_legacy":
        n_mb = B // micro_batch_size
        for i in range(n_mb):
            sl = slice(i * micro_batch_size, (i + 1) * micro_batch_size)
            out[sl] = advantages[sl] / loss_mask[sl].sum().clamp(min=1) / n_mb
        return out
    if loss_reduction == "prompt_mean":
        if prompt_boundaries is None:
            raise ValueError("`prompt_mean` loss reduction requires `prompt_boundaries`")
        P = len(prompt_boundaries)
        for s, e in prompt_boundaries:
            out[s:e] = advantages[s:e] / (P * loss_mask[s:e].sum().clamp(min=1))
        return out
    raise ValueError(f"Invalid loss reduction type: {loss_reduction}")


# ----------------------------------------------------------------------------- policy losses
def _finish(loss, old_log_probs, rollout_logprobs, loss_mask, config, metrics):
    loss, loss_mask, extra = apply_off_policy_correction(loss, old_log_probs, rollout_logprobs, loss_mask,
                                                         config.off_policy_correction)
    metrics.update(extra)
    return reduce_loss(loss, loss_mask), metrics


def _clip_frac(pred: torch.Tensor, loss_mask) -> float:
    return masked_mean(pred.float(), loss_mask).mean().detach().item()


@register_policy_loss(PolicyLossType.REGULAR)
@register_policy_loss(PolicyLossType.DUAL_CLIP)
def ppo_policy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """Clipped surrogate; ``dual_clip`` additionally bounds the loss of negative-advantage tokens."""
    assert config.policy_loss_type in ("regular", "dual_clip")
    ratio = safe_exp_delta(log_probs - old_log_probs, 20.0, log_probs.dtype)
    surr1 = ratio * advantages
    surr2 = ratio.clamp(1 - config.eps_clip_low, 1 + config.eps_clip_high) * advantages
    loss = -torch.min(surr1, surr2)
    metrics = {"clip_ratio": _clip_frac(-surr2 > -surr1, loss_mask)}
    if config.policy_loss_type == "dual_clip":
        bounded = torch.min(-advantages * config.clip_ratio_c, loss)
        loss = torch.where(advantages < 0, bounded, loss)
    return _finish(loss, old_log_probs, rollout_logprobs, loss_mask, config, metrics)


@register_policy_loss(PolicyLossType.GSPO)
def gspo_policy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """GSPO-token (https://arxiv.org/abs/2507.18071): sequence-level importance weight, token-level gradient."""
    seq_log_w = masked_mean(log_probs - old_log_probs, loss_mask, dim=-1).unsqueeze(-1)
    log_w = torch.clamp(log_probs - log_probs.detach() + seq_log_w.detach(), max=10)
    ratio = torch.exp(log_w)
    surr1 = ratio * advantages
    surr2 = ratio.clamp(1 - config.eps_clip_low, 1 + config.eps_clip_high) * advantages
    loss = -torch.min(surr1, surr2)
    metrics = {"clip_ratio": _clip_frac(-surr2 > -surr1, loss_mask)}
    return _finish(loss, old_log_probs, rollout_logprobs, loss_mask, config, metrics)


@register_policy_loss(PolicyLossType.SAPO)
def sapo_policy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """Soft adaptive policy optimisation (https://arxiv.org/abs/2511.20347): sigmoid gate instead of a hard clip."""
    ratio = torch.exp(torch.clamp(log_probs - old_log_probs, min=-20.0, max=20.0))
    tau = torch.where(advantages > 0, torch.as_tensor(config.sapo.tau_pos, dtype=advantages.dtype),
                      torch.as_tensor(config.sapo.tau_neg, dtype=advantages.dtype)).to(advantages.device)
    gates = torch.sigmoid(tau * (ratio - 1.0)) * (4.0 / tau)
    return _finish(-gates * advantages, old_log_probs, rollout_logprobs, loss_mask, config, {"clip_ratio": 0.0})


@register_policy_loss(PolicyLossType.CISPO)
def compute_policy_loss_cispo(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """CISPO (https://arxiv.org/abs/2506.13585): clip the IS weight of the gradient, not the objective."""
    if config.cispo.cispo_anchor == "rollout":
        assert rollout_logprobs is not None, "rollout_logprobs are required for cispo with cispo_anchor='rollout'"
        if config.off_policy_correction.tis_ratio_type is not None:
            raise ValueError("cispo_anchor='rollout' already performs the off-policy correction; "
                             "set off_policy_correction.tis_ratio_type=None")
        behaviour = rollout_logprobs
    else:
        behaviour = old_log_probs
    lo, hi = 1 - config.cispo.cispo_eps_clip_low, 1 + config.cispo.cispo_eps_clip_high
    ratio = safe_exp_delta(log_probs - behaviour, 20.0, log_probs.dtype)
    clamped = ratio.clamp(lo, hi)
    loss = -advantages * clamped.detach() * log_probs
    act = ratio[loss_mask.bool()] if loss_mask is not None and loss_mask.any() else ratio
    metrics = {
        "clip_ratio": _clip_frac((ratio < lo) | (ratio > hi), loss_mask),
        "cispo/ratio_mean": masked_mean(ratio, loss_mask).mean().item(),
        "cispo/ratio_clamped_mean": masked_mean(clamped, loss_mask).mean().item(),
        "cispo/ratio_max": act.max().item(),
        "cispo/ratio_min": act.min().item(),
    }
    return _finish(loss, old_log_probs, rollout_logprobs, loss_mask, config, metrics)


@register_policy_loss(PolicyLossType.ROLLOUT_IS)
def rollout_is_policy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """IS-weighted policy gradient anchored on the rollout policy; weights outside the band are zeroed."""
    assert rollout_logprobs is not None, "rollout_logprobs are required for rollout_is"
    ratio = safe_exp_delta(log_probs - rollout_logprobs, 20.0, log_probs.dtype)
    inside = (ratio > 1 - config.eps_clip_low) & (ratio < 1 + config.eps_clip_high)
    w = torch.where(inside, ratio, torch.zeros_like(ratio)).detach()
    metrics = {"clip_ratio": _clip_frac(~inside, loss_mask)}
    return _finish(-(w * advantages * log_probs), old_log_probs, rollout_logprobs, loss_mask, config, metrics)


@register_policy_loss(PolicyLossType.DPPO)
def dppo_policy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """Divergence-proximal PO (https://arxiv.org/abs/2602.04879): binary TV / KL trust-region mask."""
    mu = rollout_logprobs if rollout_logprobs is not None else old_log_probs
    ratio = safe_exp_delta(log_probs - mu, 20.0, log_probs.dtype)
    with torch.no_grad():
        p, q = torch.exp(log_probs), torch.exp(mu)
        diff = p - q
        keep = torch.ones_like(advantages)
        if config.dppo.dppo_type == "binary_tv":
            keep[(advantages > 0) & (diff > config.dppo.delta_high)] = 0.0
            keep[(advantages < 0) & (-diff > config.dppo.delta_low)] = 0.0
        elif config.dppo.dppo_type == "binary_kl":
            eps = 1e-8
            bkl = q * (mu - log_probs) + (1 - q) * torch.log((1 - q + eps) / (1 - p + eps))
            keep[(advantages > 0) & (diff > 0) & (bkl > config.dppo.delta_high)] = 0.0
            keep[(advantages < 0) & (diff < 0) & (bkl > config.dppo.delta_low)] = 0.0
        else:
            raise ValueError(f"Unknown DPPO type: {config.dppo.dppo_type}. Must be 'binary_tv' or 'binary_kl'.")
    metrics = {"clip_ratio": _clip_frac(keep == 0, loss_mask)}
    return _finish(-(ratio * advantages * keep), old_log_probs, rollout_logprobs, loss_mask, config, metrics)


@register_policy_loss(PolicyLossType.CLIP_COV)
def compute_policy_loss_clip_cov(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """Clip-Cov (Entropy-Mechanism-of-RL): drop the gradient of a random subset of high-covariance tokens."""
    ratio = torch.exp(log_probs - old_log_probs)
    l1 = -advantages * ratio
    l2 = -advantages * ratio.clamp(1 - config.eps_clip_low, 1 + config.eps_clip_high)
    clipped = (l2 > l1) & (loss_mask > 0)
    cov = (advantages - masked_mean(advantages, loss_mask)) * (log_probs - masked_mean(log_probs.detach(), loss_mask))
    cov = cov.detach().clone()
    cov[loss_mask == 0] = -torch.inf
    cov[clipped] = -torch.inf
    budget = max(int(config.clip_cov.clip_ratio * loss_mask.sum().item()), 1)
    cand = torch.nonzero((cov < config.clip_cov.clip_cov_ub) & (cov > config.clip_cov.clip_cov_lb) & (loss_mask > 0))
    corr = torch.ones_like(advantages)
    if len(cand) > 0:
        pick = cand[torch.randperm(len(cand))[: min(budget, len(cand))]]
        corr[pick[:, 0], pick[:, 1]] = 0
    frac = masked_mean((corr == 0).float(), loss_mask)
    return reduce_loss(torch.maximum(l1, l2) * corr, loss_mask), {"clip_ratio": frac.item()}


@register_policy_loss(PolicyLossType.KL_COV)
def compute_policy_loss_kl_cov(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """KL-Cov: add a KL penalty on the top-covariance fraction of tokens."""
    d = log_probs - old_log_probs
    ratio = torch.exp(d)
    base = -advantages * ratio
    with_kl = base + config.kl_cov.ppo_kl_coef * d.abs()
    losses = base.clone()
    valid = loss_mask > 0
    idx = torch.nonzero(valid.reshape(-1), as_tuple=True)[0]
    if idx.numel() > 0:
        a = advantages[valid].detach().reshape(-1).float()
        lp = log_probs[valid].detach().reshape(-1).float()
        cov = (a - a.mean()) * (lp - lp.mean())
        k = max(1, int(cov.numel() * config.kl_cov.kl_cov_frac))
        top = idx[torch.topk(cov, min(k, cov.numel()), largest=True).indices]
        R = advantages.shape[1]
        losses[top // R, top % R] = with_kl[top // R, top % R]
    return reduce_loss(losses, loss_mask), {"clip_ratio": 0.0}


@register_policy_loss(PolicyLossType.CROSS_ENTROPY)
def cross_entropy_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """SFT negative log-likelihood, summed (Tinker ``cross_entropy`` semantics)."""
    return reduce_loss(-log_probs, loss_mask), {"clip_ratio": 0.0}


@register_policy_loss(PolicyLossType.IMPORTANCE_SAMPLING)
def importance_sampling_loss(log_probs, old_log_probs, advantages, config, loss_mask=None, rollout_logprobs=None):
    """``-(exp(logp - logq) * A).sum()`` (Tinker ``importance_sampling`` semantics)."""
    ratio = torch.exp(log_probs - old_log_probs)
    loss = -(ratio * advantages)
    if loss_mask is not None:
        return (loss * loss_mask).sum(), {"importance_ratio": ((ratio * loss_mask).sum() / loss_mask.sum()).item()}
    return loss.sum(), {"importance_ratio": ratio.mean().item()}


def ppo_critic_loss(values, old_values, returns, config, loss_mask=None):
    """Clipped value loss ``0.5 * mean_seq(masked_mean_t(max((v_clip - R)^2, (v - R)^2)))``."""
    if config.value_clip is not None:
        v_clip = old_values + (values - old_values).clamp(-config.value_clip, config.value_clip)
        s1, s2 = (v_clip - returns) ** 2, (values - returns) ** 2
        loss = torch.max(s1, s2)
        clipfrac = masked_mean((s1 > s2).float(), loss_mask).mean().detach().item()
    else:
        loss, clipfrac = (values - returns) ** 2, None
    return 0.5 * masked_mean(loss, loss_mask, dim=-1).mean(), clipfrac


# ----------------------------------------------------------------------------- fused CUDA objective
_KL_CODES = {"k1": 0, "abs": 1, "k2": 2, "k3": 3}


class FusedPolicyObjective(torch.autograd.Function):
    """Clipped policy loss + KL penalty, value and gradient from one kernel pass (``sb_policy_loss``).

    Returns ``(weighted_total, stats[8])`` where ``weighted_total = w_pol * L_policy + w_kl * sum(kl_weights * KL)`` and
    stats are the raw sums documented in ``csrc/rl_loss.cu``.  Only ``log_probs`` receives a gradient.
    """

    @staticmethod
    def forward(ctx, log_probs, old_log_probs, advantages, loss_mask, ref_log_probs, tis, kl_weights, eps_low, eps_high,
                clip_c, dual_clip, kl_type, w_pol, w_kl):
        lib = _lib.kernels()
        vp, cf, ci = ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        lib.sb_policy_loss.argtypes = [vp, vp, vp, vp, vp, vp, vp, ctypes.c_longlong, cf, cf, cf, ci, ci, cf, cf, vp, vp, vp]
        lp = log_probs.float().contiguous()
        args = [t.float().contiguous() if t is not None else None for t in (old_log_probs, advantages, loss_mask,
                                                                            ref_log_probs, tis, kl_weights)]
        dlogp = torch.empty_like(lp)
        stats = torch.zeros(8, device=lp.device, dtype=torch.float32)
        code = lib.sb_policy_loss(lp.data_ptr(), args[0].data_ptr(), args[1].data_ptr(), args[2].data_ptr(),
                                  _lib.ptr(args[3]), _lib.ptr(args[4]), _lib.ptr(args[5]), lp.numel(), eps_low, eps_high,
                                  clip_c,
                                  1 if dual_clip else 0, _KL_CODES[kl_type], w_pol, w_kl, dlogp.data_ptr(),
                                  stats.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sb_policy_loss")
        ctx.save_for_backward(dlogp)
        ctx.shape = log_probs.shape
        ctx.dtype = log_probs.dtype
        ctx.mark_non_differentiable(stats)
        return w_pol * stats[0] + w_kl * stats[2], stats

    @staticmethod
    def backward(ctx, g_total, _g_stats):
        (dlogp,) = ctx.saved_tensors
        return ((dlogp * g_total).reshape(ctx.shape).to(ctx.dtype),) + (None,) * 13


def fused_objective_supported(config) -> bool:
    oc = config.off_policy_correction
    simple_off_policy = (oc.sequence_mask_metric is None and oc.outlier_token_is_threshold_low is None
                         and oc.outlier_token_is_threshold_high is None and oc.token_mask_is_threshold_low is None
                         and oc.tis_ratio_type is None)
    return config.policy_loss_type in ("regular", "dual_clip") and simple_off_policy


def off_policy_correction_enabled_cfg(algorithm_cfg) -> bool:
    from .off_policy import off_policy_correction_enabled

    return off_policy_correction_enabled(algorithm_cfg.off_policy_correction)
