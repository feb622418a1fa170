"""Run under torchrun on CPU (gloo), world size 2: host-side logic of the multi-rank paths."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel import tensor_parallel as tpm  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def check_tp(env):
    W, r = env.world_size, env.rank
    tp = tpm.TPGroup(None)
    assert not tp.fused and tp.size == W
    T, H, F = 8 * W, 16, 32
    g = torch.Generator().manual_seed(0)
    x_full, w1, w2 = torch.randn(T, H, generator=g), torch.randn(F, H, generator=g) * 0.1, torch.randn(H, F, generator=g) * 0.1
    dy = torch.randn(T, H, generator=g)
    R, Fs = T // W, F // W
    x = x_full[r * R : (r + 1) * R].clone().requires_grad_()
    w1s = w1[r * Fs : (r + 1) * Fs].clone().requires_grad_()
    w2s = w2[:, r * Fs : (r + 1) * Fs].clone().requires_grad_()
    y = tpm.row_parallel_linear(tpm.column_parallel_linear(x, w1s, None, tp), w2s, tp)
    y.backward(dy[r * R : (r + 1) * R])
    xr, w1r, w2r = x_full.clone().requires_grad_(), w1.clone().requires_grad_(), w2.clone().requires_grad_()
    yr = (xr @ w1r.t()) @ w2r.t()
    yr.backward(dy)
    assert rel(y, yr[r * R : (r + 1) * R]) < 1e-5
    assert rel(x.grad, xr.grad[r * R : (r + 1) * R]) < 1e-5
    assert rel(w1s.grad, w1r.grad[r * Fs : (r + 1) * Fs]) < 1e-5
    assert rel(w2s.grad, w2r.grad[:, r * Fs : (r + 1) * Fs]) < 1e-5


def check_sharded_optimizer(env):
    from skyrl_b200.parallel.sharded_optimizer import ShardedAdamW

    W, r = env.world_size, env.rank
    N = 64 * W
    torch.manual_seed(0)
    p = torch.randn(N)
    ref = p.clone().requires_grad_()
    opt_ref = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    grads = torch.zeros(N)
    opt = ShardedAdamW(p, grads, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1e9)
    for step in range(3):
        torch.manual_seed(10 * step + r)
        g_local = torch.randn(N)
        grads.copy_(g_local)
        g_sum = g_local.clone()
        dist.all_reduce(g_sum)
        ref.grad = g_sum
        opt.step()
        opt.zero_grad()
        opt_ref.step()
        assert rel(p, ref.detach()) < 1e-5, (step, rel(p, ref.detach()))


def check_tp_model(env):
    """Sharded model == unsharded model: hidden states, log-probs, and gradients of sharded + replicated params."""
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.models.tp_decoder import TPCausalLM, pad_packed_for_tp, shard_param
    import dataclasses

    W, r = env.world_size, env.rank
    a = dataclasses.replace(PRESETS["tiny-llama"], num_kv_heads=2, num_heads=4)
    tp = tpm.TPGroup(None)
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=3)
    m = TPCausalLM(a, tp, device="cpu", dtype=torch.float32, seed=3)
    lens = [37, 50, 20]
    ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(1)).int()
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    cu = torch.tensor([0, 37, 87, 107]).int()
    ids_p, pos_p, cu_p, T = pad_packed_for_tp(ids, pos, cu, W)
    assert ids_p.numel() % (W * 128) == 0 and cu_p[-1] == ids_p.numel()
    tgt = torch.roll(ids_p.long(), -1)
    h = m(ids_p, pos_p, cu_p, 128)
    lp, _ = m.token_logprobs_full(h, tgt)
    wts = torch.zeros(ids_p.numel())
    wts[:T] = torch.linspace(0.5, 1.5, T)
    (lp * wts).sum().backward()
    m.reduce_replicated_grads()
    hf = full(ids_p, pos_p, cu_p, 128)
    lpf, _ = full.token_logprobs(hf, tgt)
    (lpf * wts).sum().backward()
    R = ids_p.numel() // W
    assert rel(h, hf[r * R : (r + 1) * R]) < 1e-4, rel(h, hf[r * R : (r + 1) * R])
    assert rel(lp[:T], lpf[:T]) < 1e-4
    for name, prm in m.named_flat_views():
        want = shard_param(name, full.p(name).grad, a, W, r)
        assert rel(prm.grad, want) < 2e-3, (name, rel(prm.grad, want))
    st = m.gather_full_state()
    for name, _ in full.named_flat_views():
        assert torch.equal(st[name], full.p(name).detach()), name


def check_ulysses_model(env):
    """Sequence-parallel model == plain model once the weight gradients are summed over ranks."""
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.models.tp_decoder import UlyssesCausalLM, pad_packed_for_tp
    from skyrl_b200.parallel import ulysses
    import dataclasses

    W, r = env.world_size, env.rank
    sp = tpm.TPGroup(None)
    # layout exchange round trip
    x = torch.arange(3 * 16, dtype=torch.float32).reshape(3, 16) + 100 * r
    y = ulysses.seq_to_head(x, [8, 4, 4], sp)
    assert y.shape == (3 * W, 16 // W)
    assert torch.equal(ulysses.head_to_seq(y, [8, 4, 4], sp), x)
    a = dataclasses.replace(PRESETS["tiny-llama"], num_kv_heads=2, num_heads=4)
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=5)
    m = UlyssesCausalLM(a, sp, device="cpu", dtype=torch.float32, seed=5)
    lens = [30, 61]
    ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(2)).int()
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    cu = torch.tensor([0, 30, 91]).int()
    ids_p, pos_p, cu_p, T = pad_packed_for_tp(ids, pos, cu, W)
    tgt = torch.roll(ids_p.long(), -1)
    wts = torch.zeros(ids_p.numel())
    wts[:T] = 1.0
    lp, _ = m.token_logprobs_full(m(ids_p, pos_p, cu_p, 128), tgt)
    (lp * wts).sum().backward()
    lpf, _ = full.token_logprobs(full(ids_p, pos_p, cu_p, 128), tgt)
    (lpf * wts).sum().backward()
    assert rel(lp[:T], lpf[:T]) < 1e-4, rel(lp[:T], lpf[:T])
    for name, prm in m.named_flat_views():
        g = prm.grad.clone()
        dist.all_reduce(g)
        assert rel(g, full.p(name).grad) < 2e-3, (name, rel(g, full.p(name).grad))


def check_expert_parallel(env):
    """Experts sharded over ranks == all experts on every rank (forward, input / router-weight / expert grads)."""
    from skyrl_b200.models.moe import moe_ffn
    from skyrl_b200.parallel.expert_parallel import moe_ffn_ep

    W, r = env.world_size, env.rank
    ep = tpm.TPGroup(None)
    T, H, E, F, k = 24, 16, 4 * W, 8, 2
    g = torch.Generator().manual_seed(7)
    router = torch.randn(E, H, generator=g)
    wgu, wd = torch.randn(E, 2 * F, H, generator=g) * 0.2, torch.randn(E, H, F, generator=g) * 0.2
    hs = [torch.randn(T, H, generator=g) for _ in range(W)]
    El = E // W
    h = hs[r].clone().requires_grad_()
    wgu_l = wgu[r * El : (r + 1) * El].clone().requires_grad_()
    wd_l = wd[r * El : (r + 1) * El].clone().requires_grad_()
    rt = router.clone().requires_grad_()
    y = moe_ffn_ep(h, rt, wgu_l, wd_l, k, True, ep, E)
    gy = torch.randn(T, H, generator=torch.Generator().manual_seed(100 + r))
    y.backward(gy)
    # reference: every rank's tokens through the unsharded layer
    wgu_f, wd_f = wgu.clone().requires_grad_(), wd.clone().requires_grad_()
    tot_gu, tot_d = torch.zeros_like(wgu), torch.zeros_like(wd)
    for rr in range(W):
        hr = hs[rr].clone().requires_grad_()
        rtr = router.clone().requires_grad_()
        yr = moe_ffn(hr, rtr, wgu_f, wd_f, k, True)
        yr.backward(torch.randn(T, H, generator=torch.Generator().manual_seed(100 + rr)))
        if rr == r:
            assert rel(y, yr) < 1e-5, rel(y, yr)
            assert rel(h.grad, hr.grad) < 1e-4, rel(h.grad, hr.grad)
            assert rel(rt.grad, rtr.grad) < 1e-4, rel(rt.grad, rtr.grad)
    assert rel(wgu_l.grad, wgu_f.grad[r * El : (r + 1) * El]) < 1e-4
    assert rel(wd_l.grad, wd_f.grad[r * El : (r + 1) * El]) < 1e-4


def check_pipelined_wrapper(env):
    """Worker-facing pipeline wrapper: identical log-probs on every stage, backward through the chain, full-state gather."""
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.parallel.pipeline import PipelinedCausalLM, PipelineStage

    W, r = env.world_size, env.rank
    a = PRESETS["tiny-llama"]
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=21)
    stage = PipelineStage(a, r, W, device="cpu", dtype=torch.float32, seed=21)
    pm = PipelinedCausalLM(stage)
    g = torch.Generator().manual_seed(8)
    ids = torch.randint(4, a.vocab_size, (40,), generator=g).int()
    pos = torch.cat([torch.arange(15), torch.arange(25)]).int()
    cu = torch.tensor([0, 15, 40]).int()
    pred = torch.tensor([3, 4, 5, 20, 21, 38])
    tgt = ids[pred + 1].int()
    wts = torch.linspace(0.5, 1.5, pred.numel())
    lp, _ = pm.pred_logprobs(ids, pos, cu, 32, pred, tgt)
    (lp * wts).sum().backward()
    h = full(ids, pos, cu, 32)
    lpf, _ = full.token_logprobs(h[pred], tgt)
    (lpf * wts).sum().backward()
    assert rel(lp.detach(), lpf.detach()) < 1e-4, rel(lp.detach(), lpf.detach())
    for name, prm in stage.named_flat_views():
        ref = full.p(stage._full_name(name)).grad
        used = name.startswith("layers.") or (name == "embed" and stage.is_first) or (name in ("final_norm", "lm_head") and stage.is_last)
        if used:
            assert prm.grad is not None and rel(prm.grad, ref) < 2e-3, (name, rel(prm.grad, ref))
    with torch.no_grad():
        lp2, _ = pm.pred_logprobs(ids, pos, cu, 32, pred, tgt)
    assert rel(lp2, lpf.detach()) < 1e-4
    st = pm.gather_full_state()
    for name, _ in full.named_flat_views():
        assert torch.equal(st[name], full.p(name).detach()), name


def check_ep_model(env):
    """Expert-parallel model over both ranks' tokens == unsharded model over the union of the data."""
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.models.tp_decoder import EPCausalLM

    W, r = env.world_size, env.rank
    a = PRESETS["tiny-moe"]
    ep = tpm.TPGroup(None)
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=11)
    m = EPCausalLM(a, ep, device="cpu", dtype=torch.float32, seed=11)
    data = []
    for rr in range(W):
        g = torch.Generator().manual_seed(50 + rr)
        ids = torch.randint(4, a.vocab_size, (48,), generator=g).int()  # equal packed length on every rank
        pos = torch.cat([torch.arange(20), torch.arange(28)]).int()
        cu = torch.tensor([0, 20, 48]).int()
        data.append((ids, pos, cu))
    ids, pos, cu = data[r]
    lp, _ = m.token_logprobs(m(ids, pos, cu, 32), torch.roll(ids.long(), -1))
    lp.sum().backward()
    m.reduce_replicated_grads()
    for rr in range(W):
        i2, p2, c2 = data[rr]
        l2, _ = full.token_logprobs(full(i2, p2, c2, 32), torch.roll(i2.long(), -1))
        l2.sum().backward()
        if rr == r:
            assert rel(lp, l2) < 1e-4, rel(lp, l2)
    for name, prm in m.named_flat_views():
        want = m._shard(name, full.p(name).grad)
        assert prm.grad is not None and rel(prm.grad, want) < 3e-3, (name, rel(prm.grad, want))
    st = m.gather_full_state()
    for name, _ in full.named_flat_views():
        assert torch.equal(st[name], full.p(name).detach()), name


def check_pipeline(env):
    """Two pipeline stages reproduce the single-model loss and gradients over several micro-batches."""
    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.parallel.pipeline import PipelineStage, broadcast_from_last_stage, pipeline_forward_backward

    W, r = env.world_size, env.rank
    a = PRESETS["tiny-llama"]
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=9)
    stage = PipelineStage(a, r, W, device="cpu", dtype=torch.float32, seed=9)
    g = torch.Generator().manual_seed(4)
    mbs = []
    for lens in ([11, 20], [7], [16, 5, 9]):
        ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=g).int()
        pos = torch.cat([torch.arange(n) for n in lens]).int()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0))).int()
        mbs.append({"ids": ids, "pos": pos, "cu": cu, "max_seqlen": 32, "tgt": torch.roll(ids.long(), -1)})

    def loss_fn(model):
        return lambda h, mb: -model.token_logprobs(h, mb["tgt"])[0].sum()

    res = pipeline_forward_backward(stage, mbs, loss_fn(stage))
    ref_losses = []
    for mb in mbs:
        l = loss_fn(full)(full(mb["ids"], mb["pos"], mb["cu"], 32), mb)
        l.backward()
        ref_losses.append(l.detach())
    if stage.is_last:
        for a_, b_ in zip(res, ref_losses):
            assert abs(float(a_) - float(b_)) < 1e-3 * abs(float(b_)), (float(a_), float(b_))
    tot = broadcast_from_last_stage(torch.stack(res) if stage.is_last else None, (3,), torch.float32, stage)
    assert torch.allclose(tot, torch.stack(ref_losses), rtol=1e-3)
    for name, prm in stage.named_flat_views():
        fn = stage._full_name(name)
        ref = full.p(fn).grad
        if name == "embed" and not (stage.is_first or (stage.is_last and a.tie_word_embeddings)):
            assert prm.grad is None or prm.grad.abs().sum() == 0
            continue
        if name in ("final_norm", "lm_head") and not stage.is_last:
            assert prm.grad is None or prm.grad.abs().sum() == 0
            continue
        if name == "embed" and not a.tie_word_embeddings and stage.is_last and not stage.is_first:
            continue
        assert prm.grad is not None, name
        assert rel(prm.grad, ref) < 2e-3, (name, rel(prm.grad, ref))
    out = pipeline_forward_backward(stage, mbs[:1], None, forward_only=True)
    if stage.is_last:
        assert rel(out[0], full(mbs[0]["ids"], mbs[0]["pos"], mbs[0]["cu"], 32).detach()) < 1e-4


def main():
    env = pdist.init_distributed()
    assert env.world_size == 2 and env.device.type == "cpu"
    check_tp(env)
    check_sharded_optimizer(env)
    check_tp_model(env)
    check_ulysses_model(env)
    check_expert_parallel(env)
    check_pipeline(env)
    check_ep_model(env)
    check_pipelined_wrapper(env)
    dist.barrier()
    if env.rank == 0:
        print("CPU_CHECKS_OK", flush=True)
    pdist.shutdown()


if __name__ == "__main__":
    main()
