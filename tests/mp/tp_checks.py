"""Run under torchrun with 2+ GPUs: tensor-parallel linears with the collective inside the GEMM kernel, against an
unsharded fp32 reference, forward and backward; prints one timing line per rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.ops import _lib  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel import tensor_parallel as tpm  # noqa: E402
from skyrl_b200.parallel.peer import PeerContext  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    env = pdist.init_distributed()
    dev, W, r = env.device, env.world_size, env.rank
    ctx = PeerContext(dev, wait_seconds=5.0)
    tp = tpm.TPGroup(ctx)
    assert tp.fused
    T, H, F = 128 * W * 2, 512, 1024  # tokens, hidden, ffn (full sizes)
    R = T // W
    g = torch.Generator().manual_seed(0)
    x_full = (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(F, H, generator=g) * 0.05).to(torch.bfloat16)  # column-parallel: rows of w1 sharded
    w2 = (torch.randn(H, F, generator=g) * 0.05).to(torch.bfloat16)  # row-parallel: columns of w2 sharded
    dy_full = torch.randn(T, H, generator=g).to(torch.bfloat16)
    Fs = F // W
    x = x_full[r * R : (r + 1) * R].to(dev).requires_grad_()
    w1s = w1[r * Fs : (r + 1) * Fs].contiguous().to(dev).requires_grad_()
    w2s = w2[:, r * Fs : (r + 1) * Fs].contiguous().to(dev).requires_grad_()
    h = tpm.column_parallel_linear(x, w1s, None, tp)  # [T, F/W]
    y = tpm.row_parallel_linear(h, w2s, tp)  # [T/W, H]
    y.backward(dy_full[r * R : (r + 1) * R].to(dev))
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    xr = x_full.float().requires_grad_()
    w1r, w2r = w1.float().requires_grad_(), w2.float().requires_grad_()
    hr = (xr @ w1r.t()).to(torch.bfloat16).float()  # the sharded path rounds h to bf16 as well
    hr.retain_grad()
    yr = hr @ w2r.t()
    yr.backward(dy_full.float())
    assert rel(y.cpu(), yr[r * R : (r + 1) * R]) < 2e-2, rel(y.cpu(), yr[r * R : (r + 1) * R])
    dh = dy_full.float() @ w2.float()
    dx_ref = (dh.to(torch.bfloat16).float() @ w1.float())[r * R : (r + 1) * R]
    assert rel(x.grad.cpu(), dx_ref) < 3e-2, rel(x.grad.cpu(), dx_ref)
    dw1_ref = dh.t() @ x_full.float()
    dw2_ref = dy_full.float().t() @ hr
    assert rel(w1s.grad.cpu(), dw1_ref[r * Fs : (r + 1) * Fs]) < 3e-2
    assert rel(w2s.grad.cpu(), dw2_ref[:, r * Fs : (r + 1) * Fs]) < 3e-2

    # ---- whole model: sharded bf16 model on the fused kernels vs the unsharded bf16 model
    import dataclasses

    from skyrl_b200.models.decoder import PRESETS, CausalLM
    from skyrl_b200.models.tp_decoder import TPCausalLM, pad_packed_for_tp, shard_param

    a = dataclasses.replace(PRESETS["tiny-qwen2-d128"], num_heads=4, num_kv_heads=2, hidden_size=512, intermediate_size=1024)
    fullm = CausalLM(a, device=dev, dtype=torch.bfloat16, seed=3)
    m = TPCausalLM(a, tp, device=dev, dtype=torch.bfloat16, seed=3)
    lens = [137, 250, 90]
    ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(1)).int().to(dev)
    pos = torch.cat([torch.arange(n) for n in lens]).int().to(dev)
    cu = torch.tensor([0, 137, 387, 477]).int().to(dev)
    ids_p, pos_p, cu_p, Tr = pad_packed_for_tp(ids, pos, cu, W)
    tgt = torch.roll(ids_p.long(), -1)
    hs = m(ids_p, pos_p, cu_p, 512)
    lp, _ = m.token_logprobs_full(hs, tgt)
    wts = torch.zeros(ids_p.numel(), device=dev)
    wts[:Tr] = 1.0
    (lp.float() * wts).sum().backward()
    m.reduce_replicated_grads()
    hf = fullm(ids_p, pos_p, cu_p, 512)
    lpf, _ = fullm.token_logprobs(hf, tgt)
    (lpf.float() * wts).sum().backward()
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    Rm = ids_p.numel() // W
    assert rel(hs, hf[r * Rm : (r + 1) * Rm]) < 3e-2, rel(hs, hf[r * Rm : (r + 1) * Rm])
    assert (lp[:Tr].float() - lpf[:Tr].float()).abs().max() < 0.1
    for name, prm in m.named_flat_views():
        want = shard_param(name, fullm.p(name).grad, a, W, r)
        assert rel(prm.grad, want) < 8e-2, (name, rel(prm.grad, want))

    # ---- Ulysses sequence-parallel model on the fused projections vs the plain model
    from skyrl_b200.models.tp_decoder import UlyssesCausalLM

    um = UlyssesCausalLM(a, tp, device=dev, dtype=torch.bfloat16, seed=3)
    fullm.zero_grad()
    lpu, _ = um.token_logprobs_full(um(ids_p, pos_p, cu_p, 512), tgt)
    (lpu.float() * wts).sum().backward()
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    assert (lpu[:Tr].float() - lpf[:Tr].float()).abs().max() < 0.1
    (fullm.token_logprobs(fullm(ids_p, pos_p, cu_p, 512), tgt)[0].float() * wts).sum().backward()
    for name, prm in um.named_flat_views():
        g = prm.grad.float().clone()
        dist.all_reduce(g)
        assert rel(g, fullm.p(name).grad) < 8e-2, (name, rel(g, fullm.p(name).grad))

    # ---- expert-parallel MoE layer on the fused dispatch / combine GEMMs vs the unsharded layer
    from skyrl_b200.models.moe import moe_ffn
    from skyrl_b200.parallel.expert_parallel import moe_ffn_ep

    Tm, Hm, Em, Fm, km = 192, 256, 4 * W, 128, 2
    ge = torch.Generator().manual_seed(7)
    router = (torch.randn(Em, Hm, generator=ge) * 0.5).to(torch.bfloat16)
    wgu_f = (torch.randn(Em, 2 * Fm, Hm, generator=ge) * 0.05).to(torch.bfloat16)
    wd_f = (torch.randn(Em, Hm, Fm, generator=ge) * 0.05).to(torch.bfloat16)
    hs_all = [(torch.randn(Tm, Hm, generator=ge) * 0.5).to(torch.bfloat16) for _ in range(W)]
    El = Em // W
    he = hs_all[r].to(dev).requires_grad_()
    wgu_l = wgu_f[r * El : (r + 1) * El].contiguous().to(dev).requires_grad_()
    wd_l = wd_f[r * El : (r + 1) * El].contiguous().to(dev).requires_grad_()
    rt = router.to(dev).requires_grad_()
    ye = moe_ffn_ep(he, rt, wgu_l, wd_l, km, True, tp, Em)
    gy = torch.randn(Tm, Hm, generator=torch.Generator().manual_seed(100 + r)).to(torch.bfloat16).to(dev)
    ye.backward(gy)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    wgu_r, wd_r = wgu_f.to(dev).requires_grad_(), wd_f.to(dev).requires_grad_()
    for rr in range(W):
        hr = hs_all[rr].to(dev).requires_grad_()
        rtr = router.to(dev).requires_grad_()
        yr = moe_ffn(hr, rtr, wgu_r, wd_r, km, True)
        yr.backward(torch.randn(Tm, Hm, generator=torch.Generator().manual_seed(100 + rr)).to(torch.bfloat16).to(dev))
        if rr == r:
            assert rel(ye, yr) < 3e-2, rel(ye, yr)
            assert rel(he.grad, hr.grad) < 5e-2, rel(he.grad, hr.grad)
            assert rel(rt.grad, rtr.grad) < 8e-2, rel(rt.grad, rtr.grad)
    assert rel(wgu_l.grad, wgu_r.grad[r * El : (r + 1) * El]) < 5e-2
    assert rel(wd_l.grad, wd_r.grad[r * El : (r + 1) * El]) < 5e-2

    # ---- timing: fused all-gather GEMM and GEMM reduce-scatter against NCCL + plain GEMM (device time, max over ranks)
    from skyrl_b200.ops import gemm

    T2, H2, F2 = 8192, 3584, 18944  # 7B-shaped MLP
    R2, Fs2 = T2 // W, (F2 // W) // 128 * 128
    buf = tp.gather_buffer(T2, H2, "bench_x")
    buf.local.normal_()
    wc = (torch.randn(Fs2, H2, device=dev) * 0.02).to(torch.bfloat16)
    wr = (torch.randn(H2, Fs2, device=dev) * 0.02).to(torch.bfloat16)
    hloc = (torch.randn(T2, Fs2, device=dev) * 0.5).to(torch.bfloat16)
    slots = tp.slot_buffer(R2, H2, torch.bfloat16, "bench_y")
    xs = buf.local.view(T2, H2)[r * R2 : (r + 1) * R2].clone()
    outg = torch.empty(T2, Fs2, device=dev, dtype=torch.bfloat16)

    def timed(fn, iters=5):
        for _ in range(3):
            fn()
        ctx.barrier()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def fused_ag():
        ctx.barrier()
        tpm.gemm_all_gather(tp, buf, R2, wc, out=outg)

    def nccl_ag():
        full = torch.empty(T2, H2, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, xs)
        gemm.gemm_nt(full, wc, out=outg)

    def fused_rs():
        tpm.gemm_reduce_scatter(tp, hloc, wr, slots, R2)
        ctx.barrier()
        tpm.reduce_slots(slots.local.view(W, R2, H2))
        ctx.barrier(1)

    def nccl_rs():
        yfull = gemm.gemm_nt(hloc, wr)
        out = torch.empty(R2, H2, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(out, yfull)

    # Ulysses projections: fused exchange vs all_to_all + GEMM (7B attention shapes, T tokens over W ranks)
    from skyrl_b200.parallel import ulysses

    nq_, nkv_, d_ = 28, 4, 128
    widths = [nq_ * d_, nkv_ * d_, nkv_ * d_]
    Ru = T2 // W
    hq = (torch.randn(Ru, H2, device=dev) * 0.5).to(torch.bfloat16)
    wqkv = (torch.randn(sum(widths), H2, device=dev) * 0.02).to(torch.bfloat16)
    wo = (torch.randn(H2, nq_ * d_, device=dev) * 0.02).to(torch.bfloat16)
    att_loc = (torch.randn(T2, nq_ * d_ // W, device=dev) * 0.5).to(torch.bfloat16)
    ref_tp = tpm.TPGroup(None, tp.group)  # same ranks, no peer context -> all_to_all reference path

    with torch.no_grad():
        t_qkv_f = timed(lambda: ulysses.qkv_proj(hq, wqkv, None, widths, tp))
        t_qkv_r = timed(lambda: ulysses.qkv_proj(hq, wqkv, None, widths, ref_tp))
        t_o_f = timed(lambda: ulysses.o_proj(att_loc, wo, tp))
        t_o_r = timed(lambda: ulysses.o_proj(att_loc, wo, ref_tp))

    # expert-parallel MoE layer forward (30B-A3B expert shapes, 16 local experts per rank at W=8 -> Em/W here)
    Tm2, Hm2, Em2, Fm2, km2 = 8192, 2048, 16 * W, 768, 8
    rt2 = (torch.randn(Em2, Hm2, device=dev) * 0.5).to(torch.bfloat16)
    wgu2 = (torch.randn(Em2 // W, 2 * Fm2, Hm2, device=dev) * 0.02).to(torch.bfloat16)
    wd2 = (torch.randn(Em2 // W, Hm2, Fm2, device=dev) * 0.02).to(torch.bfloat16)
    he2 = (torch.randn(Tm2, Hm2, device=dev) * 0.5).to(torch.bfloat16)
    with torch.no_grad():
        t_ep_f = timed(lambda: moe_ffn_ep(he2, rt2, wgu2, wd2, km2, True, tp, Em2), iters=3)
        t_ep_r = timed(lambda: moe_ffn_ep(he2, rt2, wgu2, wd2, km2, True, ref_tp, Em2), iters=3)

    res = {"ulysses_qkv_fused_ms": t_qkv_f, "ulysses_qkv_a2a_ms": t_qkv_r, "ulysses_o_fused_ms": t_o_f, "ulysses_o_a2a_ms": t_o_r,
           "ep_moe_fused_ms": t_ep_f, "ep_moe_gather_ref_ms": t_ep_r,
           "ag_gemm_fused_ms": timed(fused_ag), "ag_gemm_nccl_ms": timed(nccl_ag), "gemm_rs_fused_ms": timed(fused_rs),
           "gemm_rs_nccl_ms": timed(nccl_rs), "world": W, "shape": [T2, H2, Fs2]}
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    fl = 2.0 * T2 * H2 * Fs2
    res["ag_gemm_fused_tflops"] = fl / res["ag_gemm_fused_ms"] / 1e9
    res["gemm_rs_fused_tflops"] = fl / res["gemm_rs_fused_ms"] / 1e9
    if r == 0:
        import json

        print("TP_CHECKS " + json.dumps(res), flush=True)
    dist.barrier()
    pdist.shutdown()


if __name__ == "__main__":
    main()
