"""RL objective kernels (csrc/rl_loss.cu) against the fp32 PyTorch formulas of skyrl_b200.algorithms.rl run on CPU."""
import math

import numpy as np
import pytest
import torch

from skyrl_b200.algorithms import rl
from skyrl_b200.config.config import AlgorithmConfig

pytestmark = pytest.mark.gpu


def _inputs(n=4099, seed=0, wide=False):
    g = torch.Generator().manual_seed(seed)
    lp = -torch.rand(n, generator=g) * 3
    span = 60.0 if wide else 1.2  # wide: some log-ratios leave the +-20 clamp
    old = lp + (torch.rand(n, generator=g) - 0.5) * span
    ref = lp + (torch.rand(n, generator=g) - 0.5) * (50.0 if wide else 1.0)
    adv = torch.randn(n, generator=g)
    mask = (torch.rand(n, generator=g) > 0.2).float()
    return lp, old, adv, mask, ref


def _cfg(**kw):
    c = AlgorithmConfig()
    for k, v in kw.items():
        setattr(c, k, v)
    return c


@pytest.mark.parametrize("dual", [False, True])
@pytest.mark.parametrize("kl", [None, "k1", "abs", "k2", "k3"])
@pytest.mark.parametrize("wide", [False, True])
def test_policy_loss_value_gradient_and_stats(dual, kl, wide):
    lp, old, adv, mask, ref = _inputs(wide=wide, seed=3 + int(dual))
    cfg = _cfg(policy_loss_type="dual_clip" if dual else "regular", eps_clip_low=0.2, eps_clip_high=0.28, clip_ratio_c=2.0)
    w_kl = 0.05 if kl else 0.0
    # ---- CPU oracle (autograd through the registered loss + KL estimator)
    lpc = lp.clone().requires_grad_(True)
    loss_c, met = rl.ppo_policy_loss(lpc[None], old[None], adv[None], cfg, loss_mask=mask[None])
    total_c = loss_c
    kl_sum = torch.zeros(())
    if kl:
        kl_tok = rl.compute_approx_kl(lpc[None], ref[None], loss_mask=mask[None], kl_estimator_type=kl)
        kl_sum = kl_tok.sum()
        total_c = total_c + w_kl * kl_sum
    total_c.backward()
    # ---- kernel
    lpg = lp.cuda().requires_grad_(True)
    total_g, stats = rl.FusedPolicyObjective.apply(lpg, old.cuda(), adv.cuda(), mask.cuda(), ref.cuda() if kl else None,
                                                   None, None, 0.2, 0.28, 2.0, dual, kl or "k3", 1.0, w_kl)
    total_g.backward()
    torch.cuda.synchronize()
    scale = max(1.0, abs(float(total_c)))
    assert abs(float(total_g) - float(total_c)) < 2e-4 * scale, (float(total_g), float(total_c))
    assert abs(float(stats[0]) - float(loss_c)) < 2e-4 * max(1.0, abs(float(loss_c)))
    assert abs(float(stats[3]) - float(mask.sum())) < 0.5
    assert abs(float(stats[1]) / float(mask.sum()) - met["clip_ratio"]) < 1e-5
    if kl:
        assert abs(float(stats[2]) - float(kl_sum)) < 2e-4 * max(1.0, abs(float(kl_sum)))
    gd = (lpg.grad.cpu() - lpc.grad).abs().max().item()
    assert gd < 2e-4 * max(1.0, lpc.grad.abs().max().item()), gd
    assert torch.equal(lpg.grad.cpu()[mask == 0], torch.zeros(int((mask == 0).sum())))


def test_policy_loss_tis_weights_and_kl_token_weights():
    lp, old, adv, mask, ref = _inputs(n=2048, seed=11)
    g = torch.Generator().manual_seed(5)
    tis = torch.rand(2048, generator=g) * 2
    klw = torch.rand(2048, generator=g)
    lpg = lp.cuda().requires_grad_(True)
    total, stats = rl.FusedPolicyObjective.apply(lpg, old.cuda(), adv.cuda(), mask.cuda(), ref.cuda(), tis.cuda(),
                                                 klw.cuda(), 0.2, 0.2, 3.0, False, "k2", 0.5, 0.3)
    total.backward()
    lpc = lp.clone().requires_grad_(True)
    r = torch.exp((lpc - old).clamp(-20, 20))
    pol = (-torch.min(r * adv, r.clamp(0.8, 1.2) * adv) * tis * mask).sum()
    klv = (0.5 * (lpc - ref) ** 2 * klw * mask).sum()
    want = 0.5 * pol + 0.3 * klv
    want.backward()
    assert abs(float(total) - float(want)) < 2e-4 * max(1.0, abs(float(want)))
    assert (lpg.grad.cpu() - lpc.grad).abs().max().item() < 2e-4 * max(1.0, lpc.grad.abs().max().item())


@pytest.mark.parametrize("mode", ["grpo", "dr_grpo", "rloo"])
def test_group_advantage_kernel(mode):
    g = torch.Generator().manual_seed(2)
    B, R = 37, 6
    rewards = torch.zeros(B, R)
    rewards[:, -1] = torch.randn(B, generator=g)
    mask = torch.ones(B, R)
    idx = np.array([i // 5 for i in range(B - 2)] + [100, 101])  # seven groups of five and two singletons
    if mode == "rloo":
        want, _ = rl.compute_rloo_outcome_advantage(rewards, mask, idx)
        gid, G = rl._dense_groups(idx)
        got = rl._group_advantage_cuda(rewards.sum(-1).cuda(), gid, G, 2, 1e-6).cpu()
        # a lone sample: the reference gives 0, the kernel leaves (s - mean) with mean 0; the estimator masks it
        cnt = torch.tensor([(idx == v).sum() for v in idx])
        got = torch.where(cnt > 1, got, torch.zeros_like(got))
        assert torch.allclose(got, want[:, -1], atol=1e-5)
        return
    norm = mode == "grpo"
    want, _ = rl.compute_grpo_outcome_advantage(rewards, mask, idx, grpo_norm_by_std=norm)
    got, _ = rl.compute_grpo_outcome_advantage(rewards.cuda(), mask.cuda(), idx, grpo_norm_by_std=norm)
    assert torch.allclose(got.cpu(), want, atol=2e-5)
    assert abs(float(got[-1, -1]) - float(rewards[-1, -1]) / (1 + 1e-6 if norm else 1.0)) < 1e-5  # singleton


@pytest.mark.parametrize("gamma,lam", [(1.0, 0.95), (0.99, 0.9), (1.0, 1.0)])
def test_gae_kernel_with_left_padding(gamma, lam):
    g = torch.Generator().manual_seed(4)
    B, R = 19, 33
    r, v = torch.randn(B, R, generator=g), torch.randn(B, R, generator=g)
    mask = torch.ones(B, R)
    for b in range(B):  # right-aligned responses: the first positions of a row are padding with zero reward / value
        k = int(torch.randint(0, R - 2, (1,), generator=g))
        mask[b, :k] = 0
        r[b, :k] = 0
        v[b, :k] = 0
    adv_c, ret_c = rl.compute_gae_advantage_return(r, v, mask, gamma=gamma, lambd=lam)
    adv_g, ret_g = rl.compute_gae_advantage_return(r.cuda(), v.cuda(), mask.cuda(), gamma=gamma, lambd=lam)
    assert torch.allclose(ret_g.cpu(), ret_c, atol=1e-4, rtol=1e-4)
    assert torch.allclose(adv_g.cpu(), adv_c, atol=1e-4, rtol=1e-4)
    # spot-check one row of the raw scan against the recurrence written out
    raw_g, _ = rl._gae_scan(r.cuda(), v.cuda(), gamma, lam)
    last = 0.0
    for t in range(R - 1, -1, -1):
        nv = float(v[0, t + 1]) if t + 1 < R else 0.0
        last = float(r[0, t]) + gamma * nv - float(v[0, t]) + gamma * lam * last
        assert math.isclose(float(raw_g[0, t]), last, rel_tol=1e-4, abs_tol=1e-4)
