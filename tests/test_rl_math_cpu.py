"""Closed-form checks of the RL mathematics: every policy loss, advantage estimator, KL estimator, loss reduction
and off-policy correction against an independent, loop-based restatement of its formula.

The specifications are the ones the reference checks in tests/train/algorithms/test_losses.py,
tests/train/algorithms/test_off_policy_correction.py and tests/backends/skyrl_train/utils/test_ppo_utils.py;
the oracles below are written from the formulas, not from the implementation under test.
"""

import math

import numpy as np
import pytest
import torch

from skyrl_b200.algorithms import off_policy, rl
from skyrl_b200.config.config import AlgorithmConfig


def _cfg(**kw):
    c = AlgorithmConfig()
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _rand(B=3, R=5, seed=0):
    g = torch.Generator().manual_seed(seed)
    lp = -torch.rand(B, R, generator=g) * 2
    old = lp + (torch.rand(B, R, generator=g) - 0.5) * 0.8
    adv = torch.randn(B, R, generator=g)
    mask = (torch.rand(B, R, generator=g) > 0.25).float()
    mask[:, 0] = 1
    return lp, old, adv, mask


# ----------------------------------------------------------------------------- KL
@pytest.mark.parametrize("kind", ["k1", "abs", "k2", "k3"])
def test_kl_estimators_match_formulas(kind):
    lp, ref, _, mask = _rand(seed=1)
    got = rl.compute_approx_kl(lp, ref, loss_mask=mask, kl_estimator_type=kind)
    for b in range(lp.shape[0]):
        for t in range(lp.shape[1]):
            d = float(lp[b, t] - ref[b, t])
            if kind == "k1":
                want = d
            elif kind == "abs":
                want = abs(d)
            elif kind == "k2":
                want = 0.5 * d * d
            else:
                x = min(max(-d, -20.0), 20.0)
                want = min(max(math.exp(x) - x - 1, -10.0), 10.0)
            want *= float(mask[b, t])
            assert abs(float(got[b, t]) - want) < 1e-5


def test_k3_is_clamped_and_never_nan():
    lp = torch.tensor([[0.0, -50.0, 30.0]])
    ref = torch.tensor([[-40.0, 0.0, 0.0]])
    k = rl.compute_approx_kl(lp, ref, kl_estimator_type="k3")
    assert torch.isfinite(k).all() and float(k.max()) <= 10.0


def test_kl_controllers():
    c = rl.AdaptiveKLController(0.1, target=0.1, horizon=100)
    c.update(0.2, n_steps=10)  # err clipped to +0.2 -> value *= 1 + 0.2 * 10 / 100
    assert abs(c.value - 0.1 * 1.02) < 1e-9
    c.update(0.0, n_steps=10)  # err clipped to -0.2
    assert abs(c.value - 0.1 * 1.02 * 0.98) < 1e-9
    f = rl.FixedKLController(0.3)
    f.update(5.0, 10)
    assert f.value == 0.3


# ----------------------------------------------------------------------------- advantage estimators
def test_grpo_advantage_groups_singleton_and_dr_grpo():
    rewards = torch.zeros(5, 4)
    rewards[:, -1] = torch.tensor([1.0, 3.0, 2.0, 6.0, 7.0])
    mask = torch.ones(5, 4)
    mask[1, 0] = 0
    idx = np.array(["a", "a", "b", "a", "c"], dtype=object)  # group b and c are singletons
    adv, ret = rl.compute_grpo_outcome_advantage(rewards, mask, idx, epsilon=1e-6)
    a = np.array([1.0, 3.0, 6.0])
    want_a = (a - a.mean()) / (a.std(ddof=1) + 1e-6)
    assert torch.allclose(adv[0], torch.full((4,), float(want_a[0])), atol=1e-5)
    assert torch.allclose(adv[3], torch.full((4,), float(want_a[2])), atol=1e-5)
    assert float(adv[1, 0]) == 0.0 and abs(float(adv[1, 1]) - want_a[1]) < 1e-5  # masked position
    # singleton: mean 0, std 1 -> advantage = score / (1 + eps)
    assert abs(float(adv[2, -1]) - 2.0 / (1 + 1e-6)) < 1e-5
    assert abs(float(adv[4, -1]) - 7.0 / (1 + 1e-6)) < 1e-5
    assert torch.equal(adv, ret)
    adv2, _ = rl.compute_grpo_outcome_advantage(rewards, mask, idx, grpo_norm_by_std=False)
    assert abs(float(adv2[0, -1]) - (1.0 - a.mean())) < 1e-5


def test_rloo_and_maxrl():
    rewards = torch.zeros(4, 3)
    rewards[:, -1] = torch.tensor([1.0, 2.0, 6.0, 5.0])
    mask = torch.ones(4, 3)
    idx = np.array([0, 0, 0, 1])
    adv, _ = rl.compute_rloo_outcome_advantage(rewards, mask, idx)
    # leave-one-out baseline: s_i - mean(others)
    assert abs(float(adv[0, 0]) - (1.0 - (2.0 + 6.0) / 2)) < 1e-5
    assert abs(float(adv[2, 0]) - (6.0 - (1.0 + 2.0) / 2)) < 1e-5
    assert float(adv[3, 0]) == 0.0  # a lone sample has no baseline
    m, _ = rl.compute_maxrl_advantage(rewards, mask, idx, epsilon=1e-6)
    assert abs(float(m[1, 0]) - (2.0 - 3.0) / (3.0 + 1e-6)) < 1e-5


def test_reinforce_pp_returns_reset_by_mask_and_gamma():
    rewards = torch.tensor([[0.0, 1.0, 0.0, 2.0], [1.0, 0.0, 0.0, 0.0]])
    mask = torch.tensor([[1.0, 1.0, 1.0, 1.0], [1.0, 1.0, 0.0, 0.0]])
    adv, ret = rl.compute_reinforce_plus_plus_outcome_advantage(rewards, mask, gamma=0.5)
    # row 0: G_3 = 2, G_2 = 1, G_1 = 1 + .5 = 1.5, G_0 = .75
    assert torch.allclose(ret[0], torch.tensor([0.75, 1.5, 1.0, 2.0]))
    assert torch.allclose(ret[1, :2], torch.tensor([1.0, 0.0]))
    live = ret[mask.bool()]
    want = (ret - live.mean()) / math.sqrt(float(live.var(unbiased=True)) + 1e-8) * mask
    assert torch.allclose(adv, want, atol=1e-5)


def _gae_oracle(r, v, gamma, lam):
    B, R = r.shape
    adv = torch.zeros_like(r)
    for b in range(B):
        last = 0.0
        for t in range(R - 1, -1, -1):
            nv = float(v[b, t + 1]) if t + 1 < R else 0.0
            delta = float(r[b, t]) + gamma * nv - float(v[b, t])
            last = delta + gamma * lam * last
            adv[b, t] = last
    return adv, adv + v


@pytest.mark.parametrize("gamma,lam", [(1.0, 1.0), (0.9, 0.95), (1.0, 0.5)])
def test_gae_scan_and_whitening(gamma, lam):
    g = torch.Generator().manual_seed(3)
    r, v = torch.randn(3, 6, generator=g), torch.randn(3, 6, generator=g)
    mask = torch.ones(3, 6)
    mask[1, :2] = 0
    raw, ret_want = _gae_oracle(r, v, gamma, lam)
    adv, ret = rl.compute_gae_advantage_return(r, v, mask, gamma=gamma, lambd=lam)
    assert torch.allclose(ret, ret_want, atol=1e-5)
    live = raw[mask.bool()]
    want = (raw - live.mean()) / math.sqrt(float(live.var(unbiased=True)) + 1e-8)
    assert torch.allclose(adv, want, atol=1e-4)


# ----------------------------------------------------------------------------- loss reductions
def test_loss_reductions():
    adv = torch.ones(4, 3)
    mask = torch.tensor([[1.0, 1, 1], [1, 1, 0], [1, 0, 0], [1, 1, 1]])
    f = rl.apply_loss_reduction_to_advantages_minibatch
    assert torch.allclose(f(adv, mask, "token_mean", 2, 3), adv / 9)
    sm = f(adv, mask, "sequence_mean", 2, 3)
    assert torch.allclose(sm[:, 0], torch.tensor([1 / 12, 1 / 8, 1 / 4, 1 / 12]))
    assert torch.allclose(f(adv, mask, "seq_mean_token_sum_norm", 2, 10), adv / 40)
    leg = f(adv, mask, "token_mean_legacy", 2, 3)
    assert torch.allclose(leg[0], torch.full((3,), 1 / 5 / 2)) and torch.allclose(leg[2], torch.full((3,), 1 / 4 / 2))
    pm = f(adv, mask, "prompt_mean", 2, 3, prompt_boundaries=[(0, 2), (2, 4)])
    assert torch.allclose(pm[0], torch.full((3,), 1 / (2 * 5))) and torch.allclose(pm[3], torch.full((3,), 1 / (2 * 4)))
    with pytest.raises(ValueError):
        f(adv, mask, "prompt_mean", 2, 3)
    with pytest.raises(ValueError):
        f(adv, mask, "nope", 2, 3)
    # a masked sum of pre-scaled losses equals the named reduction of the raw losses
    loss = torch.arange(12.0).view(4, 3)
    assert abs(float((loss * f(adv, mask, "sequence_mean", 2, 3) * mask).sum())
               - float(((loss * mask).sum(1) / mask.sum(1)).mean())) < 1e-5


# ----------------------------------------------------------------------------- policy losses
def _ppo_oracle(lp, old, adv, mask, lo, hi, dual_c=None):
    tot, clipped = 0.0, 0.0
    for b in range(lp.shape[0]):
        for t in range(lp.shape[1]):
            r = math.exp(min(max(float(lp[b, t] - old[b, t]), -20.0), 20.0))
            A = float(adv[b, t])
            s1, s2 = r * A, min(max(r, 1 - lo), 1 + hi) * A
            loss = -min(s1, s2)
            clipped += float(mask[b, t]) * (1.0 if -s2 > -s1 else 0.0)
            if dual_c is not None and A < 0:
                loss = min(-A * dual_c, loss)
            tot += loss * float(mask[b, t])
    return tot, clipped / float(mask.sum())


def test_regular_and_dual_clip_losses():
    lp, old, adv, mask = _rand(seed=5)
    old = lp + (old - lp) * 4  # make some ratios leave the clip band and the dual-clip bound bite
    cfg = _cfg(policy_loss_type="regular", eps_clip_low=0.2, eps_clip_high=0.3)
    got, m = rl.ppo_policy_loss(lp, old, adv, cfg, loss_mask=mask)
    want, _ = _ppo_oracle(lp, old, adv, mask, 0.2, 0.3)
    assert abs(float(got) - want) < 1e-4
    cfg = _cfg(policy_loss_type="dual_clip", eps_clip_low=0.2, eps_clip_high=0.3, clip_ratio_c=1.5)
    got, _ = rl.ppo_policy_loss(lp, old, adv, cfg, loss_mask=mask)
    want, _ = _ppo_oracle(lp, old, adv, mask, 0.2, 0.3, dual_c=1.5)
    assert abs(float(got) - want) < 1e-4


def test_ppo_gradient_is_zero_on_clipped_side():
    lp = torch.tensor([[0.0, 0.0]], requires_grad=True)
    old = torch.tensor([[-1.0, 1.0]])  # ratios e, 1/e
    adv = torch.tensor([[1.0, -1.0]])  # positive adv at a high ratio and negative adv at a low ratio: both clipped
    loss, _ = rl.ppo_policy_loss(lp, old, adv, _cfg(), loss_mask=torch.ones(1, 2))
    loss.backward()
    assert torch.equal(lp.grad, torch.zeros(1, 2))


def test_gspo_sequence_level_ratio():
    lp, old, adv, mask = _rand(seed=7)
    lpg = lp.clone().requires_grad_(True)
    cfg = _cfg(policy_loss_type="gspo")
    got, _ = rl.gspo_policy_loss(lpg, old, adv, cfg, loss_mask=mask)
    tot = 0.0
    for b in range(lp.shape[0]):
        n = float(mask[b].sum())
        s = float(((lp[b] - old[b]) * mask[b]).sum()) / n
        r = math.exp(min(s, 10.0))
        for t in range(lp.shape[1]):
            A = float(adv[b, t])
            tot += -min(r * A, min(max(r, 0.8), 1.2) * A) * float(mask[b, t])
    assert abs(float(got) - tot) < 1e-4
    got.backward()
    assert torch.isfinite(lpg.grad).all()


def test_cispo_old_and_rollout_anchor():
    lp, old, adv, mask = _rand(seed=9)
    roll = old + 0.3
    cfg = _cfg(policy_loss_type="cispo")
    cfg.cispo.cispo_eps_clip_low, cfg.cispo.cispo_eps_clip_high = 0.1, 0.2
    lpg = lp.clone().requires_grad_(True)
    got, m = rl.compute_policy_loss_cispo(lpg, old, adv, cfg, loss_mask=mask)
    want = 0.0
    for b in range(lp.shape[0]):
        for t in range(lp.shape[1]):
            r = math.exp(float(lp[b, t] - old[b, t]))
            want += -float(adv[b, t]) * min(max(r, 0.9), 1.2) * float(lp[b, t]) * float(mask[b, t])
    assert abs(float(got) - want) < 1e-4
    got.backward()  # the clipped weight is a constant: d loss / d logp = -A * clamp(r)
    r00 = math.exp(float(lp[0, 0] - old[0, 0]))
    assert abs(float(lpg.grad[0, 0]) + float(adv[0, 0]) * min(max(r00, 0.9), 1.2)) < 1e-5
    act = torch.exp(lp - old)[mask.bool()]
    assert abs(m["cispo/ratio_max"] - float(act.max())) < 1e-5 and abs(m["cispo/ratio_min"] - float(act.min())) < 1e-5
    cfg.cispo.cispo_anchor = "rollout"
    got2, _ = rl.compute_policy_loss_cispo(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=roll)
    want2 = sum(-float(adv[b, t]) * min(max(math.exp(float(lp[b, t] - roll[b, t])), 0.9), 1.2) * float(lp[b, t])
                * float(mask[b, t]) for b in range(3) for t in range(5))
    assert abs(float(got2) - want2) < 1e-4
    with pytest.raises(AssertionError):
        rl.compute_policy_loss_cispo(lp, old, adv, cfg, loss_mask=mask)
    cfg.off_policy_correction.tis_ratio_type = "token"
    with pytest.raises(ValueError):
        rl.compute_policy_loss_cispo(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=roll)


def test_rollout_is_zeroes_weights_outside_band():
    lp = torch.tensor([[0.0, 0.0, 0.0]])
    roll = torch.tensor([[0.0, -1.0, 0.1]])  # ratios 1, e (outside), 0.905 (inside)
    adv = torch.tensor([[2.0, 2.0, 2.0]])
    cfg = _cfg(policy_loss_type="rollout_is")
    lpg = lp.clone().requires_grad_(True)
    loss, m = rl.rollout_is_policy_loss(lpg, lp, adv, cfg, loss_mask=torch.ones(1, 3), rollout_logprobs=roll)
    loss.backward()
    assert torch.allclose(lpg.grad, torch.tensor([[-2.0, 0.0, -2.0 * math.exp(-0.1)]]), atol=1e-5)
    assert abs(m["clip_ratio"] - 1 / 3) < 1e-6


@pytest.mark.parametrize("kind", ["binary_tv", "binary_kl"])
def test_dppo_masks(kind):
    lp = torch.log(torch.tensor([[0.6, 0.2, 0.5, 0.5]]))
    mu = torch.log(torch.tensor([[0.3, 0.5, 0.45, 0.55]]))
    adv = torch.tensor([[1.0, -1.0, 1.0, -1.0]])
    cfg = _cfg(policy_loss_type="dppo")
    cfg.dppo.dppo_type, cfg.dppo.delta_high, cfg.dppo.delta_low = kind, 0.1, 0.1
    loss, m = rl.dppo_policy_loss(lp, mu, adv, cfg, loss_mask=torch.ones(1, 4), rollout_logprobs=mu)
    # tokens 0 and 1 moved by 0.3 in probability in the direction the advantage pushes: dropped under both measures
    ratios = torch.exp(lp - mu)
    want = -(ratios[0, 2] * 1.0) - (ratios[0, 3] * -1.0)
    assert abs(float(loss) - float(want)) < 1e-5
    assert abs(m["clip_ratio"] - 0.5) < 1e-6


def test_sapo_gate():
    lp, old, adv, mask = _rand(seed=11)
    cfg = _cfg(policy_loss_type="sapo")
    cfg.sapo.tau_pos, cfg.sapo.tau_neg = 1.0, 2.0
    got, _ = rl.sapo_policy_loss(lp, old, adv, cfg, loss_mask=mask)
    want = 0.0
    for b in range(3):
        for t in range(5):
            r = math.exp(float(lp[b, t] - old[b, t]))
            tau = 1.0 if float(adv[b, t]) > 0 else 2.0
            gate = 1 / (1 + math.exp(-tau * (r - 1))) * 4 / tau
            want += -gate * float(adv[b, t]) * float(mask[b, t])
    assert abs(float(got) - want) < 1e-4


def test_clip_cov_and_kl_cov():
    torch.manual_seed(0)
    lp, old, adv, mask = _rand(B=4, R=8, seed=13)
    cfg = _cfg(policy_loss_type="clip_cov")
    cfg.clip_cov.clip_ratio, cfg.clip_cov.clip_cov_lb, cfg.clip_cov.clip_cov_ub = 0.2, -100.0, 100.0
    loss, m = rl.compute_policy_loss_clip_cov(lp, old, adv, cfg, loss_mask=mask)
    budget = max(int(0.2 * float(mask.sum())), 1)
    assert 0 < m["clip_ratio"] <= budget / float(mask.sum()) + 1e-6 and torch.isfinite(loss)
    cfg = _cfg(policy_loss_type="kl_cov")
    cfg.kl_cov.kl_cov_frac, cfg.kl_cov.ppo_kl_coef = 0.25, 2.0
    loss, _ = rl.compute_policy_loss_kl_cov(lp, old, adv, cfg, loss_mask=mask)
    live = mask.bool()
    a, l = adv[live], lp[live]
    cov = (a - a.mean()) * (l - l.mean())
    k = max(1, int(cov.numel() * 0.25))
    top = torch.topk(cov, k).indices
    base = (-adv * torch.exp(lp - old))[live]
    pen = torch.zeros_like(base)
    pen[top] = 2.0 * (lp - old).abs()[live][top]
    assert abs(float(loss) - float((base + pen).sum())) < 1e-4


def test_cross_entropy_and_importance_sampling():
    lp, old, adv, mask = _rand(seed=15)
    ce, _ = rl.cross_entropy_loss(lp, None, None, _cfg(), loss_mask=mask)
    assert abs(float(ce) + float((lp * mask).sum())) < 1e-5
    isl, m = rl.importance_sampling_loss(lp, old, adv, _cfg(), loss_mask=mask)
    assert abs(float(isl) + float((torch.exp(lp - old) * adv * mask).sum())) < 1e-5


def test_critic_loss_clipped():
    v = torch.tensor([[1.0, 2.0, 0.0]])
    old = torch.tensor([[0.0, 2.0, 0.0]])
    ret = torch.tensor([[2.0, 1.0, 0.0]])
    mask = torch.tensor([[1.0, 1.0, 0.0]])
    loss, frac = rl.ppo_critic_loss(v, old, ret, _cfg(value_clip=0.2), loss_mask=mask)
    # token 0: v_clip = 0.2 -> (0.2-2)^2 = 3.24 > (1-2)^2; token 1: both 1
    assert abs(float(loss) - 0.5 * (3.24 + 1.0) / 2) < 1e-5 and abs(frac - 0.5) < 1e-6
    loss, frac = rl.ppo_critic_loss(v, old, ret, _cfg(value_clip=None), loss_mask=mask)
    assert abs(float(loss) - 0.5 * (1.0 + 1.0) / 2) < 1e-5 and frac is None


# ----------------------------------------------------------------------------- registries
def test_registries():
    assert set(rl.PolicyLossRegistry.list_available()) >= {"regular", "dual_clip", "gspo", "cispo", "rollout_is", "dppo",
                                                            "clip_cov", "kl_cov", "sapo", "cross_entropy",
                                                            "importance_sampling"}
    assert set(rl.AdvantageEstimatorRegistry.list_available()) >= {"grpo", "gae", "rloo", "reinforce++", "maxrl"}

    def mine(**kw):
        return None

    rl.AdvantageEstimatorRegistry.register("mine_test", mine)
    assert rl.AdvantageEstimatorRegistry.get("mine_test") is mine
    with pytest.raises(ValueError):
        rl.AdvantageEstimatorRegistry.register("mine_test", lambda **kw: None)
    rl.AdvantageEstimatorRegistry.unregister("mine_test")
    with pytest.raises(ValueError):
        rl.AdvantageEstimatorRegistry.get("mine_test")
    with pytest.raises(ValueError):
        rl.PolicyLossRegistry.unregister("never_there")


# ----------------------------------------------------------------------------- off-policy correction
def _oc(**kw):
    c = AlgorithmConfig().off_policy_correction
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def test_tis_token_and_sequence():
    old = torch.log(torch.tensor([[0.5, 0.4, 0.9], [0.2, 0.2, 0.2]]))
    roll = torch.log(torch.tensor([[0.25, 0.4, 0.3], [0.4, 0.1, 0.2]]))
    mask = torch.tensor([[1.0, 1.0, 1.0], [1.0, 1.0, 0.0]])
    c = _oc(tis_ratio_type="token", token_tis_ratio_clip_high=2.5)
    r, m = off_policy.compute_tis_ratio(old, roll, mask, "token", c)
    assert torch.allclose(r, torch.tensor([[2.0, 1.0, 2.5], [0.5, 2.0, 1.0]]), atol=1e-5)
    assert abs(m["tis_token_clip_high_ratio"] - 1 / 5) < 1e-6
    c = _oc(tis_ratio_type="sequence", sequence_tis_ratio_clip_high=5.0)
    r, m = off_policy.compute_tis_ratio(old, roll, mask, "sequence", c)
    assert torch.allclose(r.squeeze(-1), torch.tensor([5.0, 1.0]), atol=1e-5)  # 2*1*3 = 6 capped; .5*2 = 1 (masked out)
    assert abs(m["tis_seq_clip_high_ratio"] - 0.5) < 1e-6
    with pytest.raises(ValueError):
        off_policy.compute_tis_ratio(old, roll, mask, "nope", c)


def test_sequence_masks_geometric_and_product():
    old = torch.log(torch.tensor([[0.5, 0.5], [0.9, 0.9], [0.1, 0.1]]))
    roll = torch.log(torch.tensor([[0.5, 0.5], [0.3, 0.3], [0.4, 0.4]]))
    mask = torch.ones(3, 2)
    c = _oc(sequence_mask_metric="geometric", geo_mask_high=2.0, geo_mask_low=0.5)
    keep, m = off_policy.compute_sequence_mask(old, roll, mask, "geometric", c)
    assert keep.squeeze(-1).tolist() == [1.0, 0.0, 0.0]  # geometric means 1, 3, 0.25
    assert abs(m["geo_sequence_mask_over_high_ratio"] - 1 / 3) < 1e-6
    c = _oc(sequence_mask_metric="product", product_mask_high=10.0, product_mask_low=0.1)
    keep, m = off_policy.compute_sequence_mask(old, roll, mask, "product", c)
    assert keep.squeeze(-1).tolist() == [1.0, 1.0, 0.0]  # products 1, 9, 1/16
    with pytest.raises(ValueError):
        off_policy.compute_sequence_mask(old, roll, mask, "nope", c)


def test_outlier_and_token_masks():
    old = torch.log(torch.tensor([[0.5, 0.5, 0.5], [0.5, 0.9, 0.5], [0.5, 0.05, 0.5]]))
    roll = torch.log(torch.tensor([[0.5, 0.5, 0.5], [0.5, 0.1, 0.5], [0.5, 0.5, 0.5]]))
    mask = torch.tensor([[1.0, 1, 1], [1, 1, 1], [1, 0, 1]])
    c = _oc(outlier_token_is_threshold_low=0.2, outlier_token_is_threshold_high=5.0)
    keep, m = off_policy.compute_outlier_token_mask(old, roll, mask, c)
    assert keep.squeeze(-1).tolist() == [1.0, 0.0, 1.0]  # row 2's outlier is a masked-out token: kept
    c = _oc(outlier_token_is_threshold_low=None, outlier_token_is_threshold_high=5.0)
    assert off_policy.compute_outlier_token_mask(old, roll, torch.ones(3, 3), c)[0].squeeze(-1).tolist() == [1.0, 0.0, 1.0]
    c = _oc(token_mask_is_threshold_low=0.5, token_mask_is_threshold_high=2.0)
    tm, m = off_policy.compute_token_mask(old, roll, mask, c)
    assert tm.tolist() == [[1.0, 1, 1], [1, 0, 1], [1, 1, 1]]
    assert abs(m["token_mask_ratio"] - 1 / 8) < 1e-6


def test_off_policy_correction_composes_and_feeds_ppo_loss():
    lp, old, adv, mask = _rand(seed=21)
    roll = old - 0.2
    c0 = _oc()
    assert off_policy.compute_off_policy_correction(old, roll, mask, c0) == (None, {}, mask)
    cfg = _cfg(policy_loss_type="regular")
    cfg.off_policy_correction.tis_ratio_type = "token"
    cfg.off_policy_correction.token_tis_ratio_clip_high = 1.1
    cfg.off_policy_correction.sequence_mask_metric = "geometric"
    cfg.off_policy_correction.geo_mask_high, cfg.off_policy_correction.geo_mask_low = 1.5, 0.5
    got, m = rl.ppo_policy_loss(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=roll)
    base = -torch.min(torch.exp(lp - old) * adv, torch.exp(lp - old).clamp(0.8, 1.2) * adv)
    tis = torch.exp(old - roll).clamp(max=1.1)
    assert abs(float(got) - float((base * tis * mask).sum())) < 1e-4  # exp(0.2) = 1.22 geometric mean: all kept
    assert "is_ratio_mean" in m and "tis_token_clip_high_ratio" in m
    cfg.off_policy_correction.geo_mask_high = 1.1  # now every sequence is rejected
    got, _ = rl.ppo_policy_loss(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=roll)
    assert float(got) == 0.0


def test_chunked_entropy_helpers_for_code_written_against_logits():
    import math

    from skyrl_b200.utils.torch_utils import chunked_cross_entropy_from_log_probs, chunked_entropy_from_logits

    logits = torch.tensor([[[1.0, 2.0, 3.0, 4.0], [1.0, 0.0, 0.0, 0.0], [0.0, 0.0, 0.0, 0.0]],
                           [[0.0, 0.0, 0.0, 0.0], [1.0, 2.0, 3.0, 4.0], [4.0, 3.0, 2.0, 1.0]]])
    for got in (chunked_entropy_from_logits(logits, chunk=2), chunked_cross_entropy_from_log_probs(torch.log_softmax(logits, -1), chunk=2)):
        assert got.shape == (2, 3) and torch.allclose(got[0, 2], torch.tensor(math.log(4.0)), atol=1e-4)
        assert torch.allclose(got[1, 0], torch.tensor(math.log(4.0)), atol=1e-4) and torch.allclose(got[0, 0], got[1, 1])
    x = torch.randn(2, 4, 4)
    mask = torch.tensor([[1, 1, 1, 1], [1, 1, 0, 0]], dtype=torch.float32)
    masked, free = chunked_entropy_from_logits(x, attention_mask=mask), chunked_entropy_from_logits(x)
    assert masked[1, 2] == 0 and masked[1, 3] == 0 and torch.allclose(masked[0], free[0]) and torch.allclose(masked[1, :2], free[1, :2])
    for bad in (torch.ones(3, 4), torch.ones(2, 5)):
        with pytest.raises(ValueError, match="does not match logits shape"):
            chunked_entropy_from_logits(x, attention_mask=bad)
    y = torch.randn(1, 3, 5, requires_grad=True)
    assert not chunked_entropy_from_logits(y).requires_grad and chunked_entropy_from_logits(y, requires_grad=True).requires_grad
