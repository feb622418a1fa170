"""Elementwise, attention, decode, sampling and optimizer kernels against fp32 PyTorch references."""
import math

import pytest
import torch

from skyrl_b200.ops import _lib, attention, elementwise, optim, sampling

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("T,H", [(7, 256), (1000, 1536), (333, 3584), (4099, 2048), (65, 768), (513, 264)])
def test_add_rmsnorm_fwd_bwd(T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    d = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    xn, y = elementwise.add_rmsnorm(x, d, w, 1e-6)
    g1, g2 = torch.randn_like(xn), torch.randn_like(y)
    (xn * g1).sum().backward(retain_graph=True)
    (y * g2).sum().backward()
    xr, dr, wr = (t.detach().float().requires_grad_() for t in (x, d, w))
    s = (xr + dr).to(torch.bfloat16).float() + 0 * (xr + dr)  # rounding point as in the kernel
    s = xr + dr
    yr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((s * g1.float()).sum() + (yr * g2.float()).sum()).backward()
    assert rel(xn, s) < 5e-3 and rel(y, yr) < 8e-3
    assert rel(x.grad, xr.grad) < 1e-2 and rel(d.grad, dr.grad) < 1e-2 and rel(w.grad, wr.grad) < 1e-2


def test_rope_roundtrip_and_ref():
    torch.manual_seed(0)
    T, nq, nkv, D = 300, 12, 2, 128
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    tab = elementwise.build_rope_table(4096, D, 1e6, "cuda")
    ref = elementwise._rope_ref(qkv.cpu(), pos.cpu(), tab.cpu(), nq + nkv, D, 1.0)
    got = elementwise.rope_(qkv.clone(), pos, tab, nq + nkv, D, 1.0)
    assert rel(got.cpu(), ref) < 5e-3
    back = elementwise.rope_(got.clone(), pos, tab, nq + nkv, D, -1.0)
    assert rel(back, qkv) < 1e-2
    assert torch.equal(got[:, (nq + nkv) * D:], qkv[:, (nq + nkv) * D:])


def test_swiglu():
    torch.manual_seed(0)
    gu = torch.randn(513, 2 * 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = elementwise.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    r = gu.detach().float().requires_grad_()
    o = torch.nn.functional.silu(r[:, :1024]) * r[:, 1024:]
    o.backward(g.float())
    assert rel(out, o) < 5e-3 and rel(gu.grad, r.grad) < 8e-3


def _mk_qkv(lens, nq, nkv, D=128, seed=0):
    torch.manual_seed(seed)
    T = sum(lens)
    qkv = (torch.randn(T, (nq + 2 * nkv) * D, device="cuda") * 0.7).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    return qkv, cu


@pytest.mark.parametrize("lens,nq,nkv", [([128], 2, 1), ([64], 2, 2), ([300, 17, 129, 512], 12, 2), ([1000, 1], 4, 4)])
def test_attn_fwd(lens, nq, nkv):
    qkv, cu = _mk_qkv(lens, nq, nkv)
    out = attention.attn_varlen(qkv, cu, nq, nkv, 128)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    ref, _ = attention.attn_varlen_ref(qkv, cu, nq, nkv, 128, 1 / math.sqrt(128))
    assert rel(out, ref) < 1e-2


@pytest.mark.parametrize("lens,nq,nkv", [([128], 2, 1), ([64], 2, 2), ([300, 17, 129, 512], 12, 2), ([700, 1], 4, 4)])
def test_attn_bwd(lens, nq, nkv):
    qkv, cu = _mk_qkv(lens, nq, nkv, seed=1)
    qkv.requires_grad_()
    out = attention.attn_varlen(qkv, cu, nq, nkv, 128)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    x = qkv.detach().float().requires_grad_()
    ref, _ = attention.attn_varlen_ref(x, cu, nq, nkv, 128, 1 / math.sqrt(128))
    ref.backward(g.float())
    D = 128
    for name, sl in (("dq", slice(0, nq * D)), ("dk", slice(nq * D, (nq + nkv) * D)), ("dv", slice((nq + nkv) * D, None))):
        assert rel(qkv.grad[:, sl], x.grad[:, sl]) < 2e-2, name


def test_attn_fwd_bwd_with_drifting_row_maxima():
    """Scores whose row maximum keeps growing along the sequence (and by different amounts per row) force the forward
    kernel to move its softmax reference after the first key/value block, for some rows of a warp and not for others:
    the accumulator in tensor memory is rescaled mid-sequence.  Output, log-sum-exp (through the backward pass) and
    gradients must still match the fp32 reference."""
    torch.manual_seed(3)
    nq, nkv, D = 4, 2, 128
    lens = [700, 45, 260]
    T = sum(lens)
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device="cuda") * 0.5
    ramp = torch.linspace(0.5, 6.0, T, device="cuda")[:, None]          # keys late in a sequence score higher ...
    rows = (1.0 + 3.0 * torch.rand(T, 1, device="cuda"))                # ... by a different factor for every query row
    qkv[:, : nq * D] *= rows
    qkv[:, nq * D : (nq + nkv) * D] *= ramp
    qkv = qkv.to(torch.bfloat16).requires_grad_()
    cu = torch.tensor([0, 700, 745, 1005], device="cuda", dtype=torch.int32)
    out = attention.attn_varlen(qkv, cu, nq, nkv, D)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    x = qkv.detach().float().requires_grad_()
    ref, _ = attention.attn_varlen_ref(x, cu, nq, nkv, D, 1 / math.sqrt(D))
    ref.backward(g.float())
    assert rel(out, ref) < 1e-2
    assert rel(qkv.grad, x.grad) < 3e-2


def test_attn_q_begin_skips_key_value_only_rows_forward_and_backward():
    """Rows before ``q_begin`` of a sequence serve as keys / values only (a cached prefix, another rank's tokens).  With
    their queries zeroed and their output gradients zero, the kernels that skip those query blocks must give the same
    output rows, dK / dV (all rows) and dQ (query rows) as the run that computes everything."""
    torch.manual_seed(5)
    nq, nkv, D = 4, 2, 128
    lens, begin = [700, 260, 130, 90], [384, 0, 129, 64]   # block-aligned, none, one past a block, inside the first block
    T = sum(lens)
    cu = torch.tensor([0, 700, 960, 1090, 1180], device="cuda", dtype=torch.int32)
    qb = torch.tensor(begin, device="cuda", dtype=torch.int32)
    base = torch.randn(T, (nq + 2 * nkv) * D, device="cuda") * 0.6
    live = torch.ones(T, dtype=torch.bool, device="cuda")
    s0 = 0
    for n, b in zip(lens, begin):
        live[s0: s0 + b] = False
        s0 += n
    base[~live, : nq * D] = 0.0
    g = torch.randn(T, nq * D, device="cuda").to(torch.bfloat16)
    g[~live] = 0
    res = []
    for use in (False, True):
        qkv = base.to(torch.bfloat16).requires_grad_()
        out = attention.attn_varlen(qkv, cu, nq, nkv, D, q_begin=qb if use else None)
        out.backward(g)
        torch.cuda.synchronize()
        assert _lib.status_read_clear() == 0
        res.append((out.detach().float(), qkv.grad.float()))
    (o0, g0), (o1, g1) = res
    assert rel(o1[live], o0[live]) < 1e-3
    assert rel(g1[:, nq * D:], g0[:, nq * D:]) < 5e-3                 # dK, dV of every row
    assert rel(g1[live][:, : nq * D], g0[live][:, : nq * D]) < 5e-3   # dQ of the query rows
    # whole skipped blocks stay zero (the first 384 rows of sequence 0 are three such blocks)
    assert float(o1[:384].abs().max()) == 0.0 and float(g1[:384, : nq * D].abs().max()) == 0.0
    x = base.float().requires_grad_()
    ref, _ = attention.attn_varlen_ref(x, cu, nq, nkv, D, 1 / math.sqrt(D))
    assert rel(o1[live], ref[live]) < 1e-2


@pytest.mark.parametrize("nq,nkv,bs", [(12, 2, 16), (28, 4, 32), (4, 4, 16)])
def test_decode_paged(nq, nkv, bs):
    torch.manual_seed(0)
    D, n = 128, 5
    ctx = torch.tensor([1, 17, 300, 1025, 64], dtype=torch.int32)
    max_blocks = (int(ctx.max()) + bs - 1) // bs
    nblocks = n * max_blocks + 3
    kc = torch.randn(nblocks, bs, nkv, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(nblocks, bs, nkv, D, device="cuda").to(torch.bfloat16)
    bt = torch.randperm(nblocks)[: n * max_blocks].view(n, max_blocks).to(torch.int32).cuda()
    qkv = torch.randn(n, (nq + 2 * nkv) * D, device="cuda").to(torch.bfloat16)
    ref = attention.attn_decode_paged_ref(qkv[:, : nq * D].view(n, nq, D), kc, vc, bt, ctx, 1 / math.sqrt(D))
    for max_ctx in (0, 2048):
        for simt in (False, True):
            out = attention.attn_decode_paged(qkv, kc, vc, bt, ctx.cuda(), nq, nkv, D, max_ctx=max_ctx, force_simt=simt)
            torch.cuda.synchronize()
            assert _lib.status_read_clear() == 0
            assert rel(out.view(n, nq, D), ref) < 1e-2, (max_ctx, simt)


@pytest.mark.parametrize("n,nkv,nq", [(100, 2, 12), (160, 2, 4), (75, 4, 8)])
def test_decode_paged_many_sequences(n, nkv, nq):
    """More (sequence, kv head) pairs than SMs (several items per persistent CTA), ragged contexts, inactive slots."""
    torch.manual_seed(n)
    D, bs = 128, 32
    ctx = torch.randint(1, 700, (n,), dtype=torch.int32)
    ctx[3] = 0  # an inactive slot
    ctx[-1] = 1
    max_blocks = (int(ctx.max()) + bs - 1) // bs
    nblocks = n * max_blocks + 1
    kc = torch.randn(nblocks, bs, nkv, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(nblocks, bs, nkv, D, device="cuda").to(torch.bfloat16)
    bt = torch.randperm(nblocks)[: n * max_blocks].view(n, max_blocks).to(torch.int32).cuda()
    qkv = torch.randn(n, (nq + 2 * nkv) * D, device="cuda").to(torch.bfloat16)
    ref = attention.attn_decode_paged_ref(qkv[:, : nq * D].view(n, nq, D), kc, vc, bt, ctx, 1 / math.sqrt(D))
    out = attention.attn_decode_paged(qkv, kc, vc, bt, ctx.cuda(), nq, nkv, D, max_ctx=int(ctx.max()))
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    live = ctx > 0
    assert rel(out.view(n, nq, D)[live.cuda()], ref[live]) < 1e-2
    assert out.view(n, nq, D)[3].abs().max() == 0


def test_kv_cache_write():
    nq, nkv, D, T = 4, 2, 128, 37
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device="cuda").to(torch.bfloat16)
    kc = torch.zeros(8, 16, nkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(128)[:T].to(torch.int32).cuda()
    slots[3] = -1
    attention.kv_cache_write(qkv, kc, vc, slots, nq, nkv, D)
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    for t in (0, 5, 36):
        assert torch.equal(kc.view(-1, nkv, D)[slots[t]], k[t])
    assert kc.view(-1, nkv, D).abs().sum(dim=(1, 2)).ne(0).sum() == T - 1


def test_sampling_distribution_and_logprob():
    torch.manual_seed(0)
    V, n = 1000, 4096
    base = torch.randn(V, device="cuda") * 2
    logits = base.expand(n, V).contiguous().to(torch.bfloat16)
    temp = torch.full((n,), 0.8, device="cuda")
    tok, lp = sampling.sample(logits, temp, seed=123)
    ref_lp = torch.log_softmax(logits[0].float() / 0.8, -1)
    assert torch.allclose(lp, ref_lp[tok.long()], atol=2e-3)
    emp = torch.bincount(tok.long(), minlength=V).float() / n
    top = ref_lp.exp().topk(5).indices
    assert torch.allclose(emp[top], ref_lp.exp()[top], atol=0.03)
    tok2, _ = sampling.sample(logits, torch.zeros(n, device="cuda"), seed=1)
    assert (tok2.long() == logits[0].float().argmax()).all()


def test_adamw_flat_matches_torch():
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    master, m, v = p.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    bf = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in (1, 2, 3):
        ref.grad = g.clone()
        opt.step()
        optim.adamw_flat(master, m, v, g, bf, 1e-3, 0.9, 0.95, 1e-8, 0.01, step)
    assert torch.allclose(master, ref.detach(), atol=1e-5, rtol=1e-5)
    assert rel(bf, master) < 5e-3
    sq = torch.zeros(1, device="cuda")
    optim.sqnorm_accum(g, sq)
    assert abs(sq.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4


# ------------------------------------------------------------------ split-K GEMM + fused partial-sum consumers
@pytest.mark.parametrize("M,N,K,splits,bn", [(256, 1536, 8960, 6, 128), (64, 2048, 1536, 4, 64), (200, 1536, 1536, 6, 128),
                                             (8, 2048, 1536, 24, 64), (130, 520, 200, 3, 64)])
def test_gemm_splitk_partials_sum_to_product(M, N, K, splits, bn):
    from skyrl_b200.ops import gemm

    torch.manual_seed(1)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device="cuda").to(torch.bfloat16)
    part = torch.full((splits, M, N), float("nan"), device="cuda")
    used = gemm.gemm_nt_splitk(x, w, b, part, splits, bn)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    assert 1 <= used <= splits
    ref = x.float() @ w.float().t() + b.float()
    got = part[:used].sum(0)
    assert torch.isfinite(got).all()
    assert ((got - ref).norm() / ref.norm()).item() < 2e-3


def test_plan_splitk_covers_the_machine_without_empty_slices():
    from skyrl_b200.ops import gemm

    for M, N, K in [(256, 2048, 1536), (256, 1536, 1536), (256, 1536, 8960), (64, 2048, 1536), (8, 1536, 8960),
                    (256, 17920, 1536), (1024, 2048, 1536)]:
        s, bn = gemm.plan_splitk(M, N, K)
        kb = (K + 63) // 64
        kpb = (kb + s - 1) // s
        assert (s - 1) * kpb < kb  # the last slice is not empty
        tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
        assert tiles * s >= 96 or s == 1 and tiles >= 96 or kb < 8


def test_add_rmsnorm_partials_matches_reference():
    from skyrl_b200.ops import elementwise as ew

    torch.manual_seed(2)
    T, H, P = 77, 1536, 5
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    part = torch.randn(P + 1, T, H, device="cuda") * 0.3
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    x_ref = (x.float() + part[:P].sum(0)).to(torch.bfloat16)
    xf = x_ref.float()
    y_ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    y = ew.add_rmsnorm_partials_(x, part, P, w, 1e-6)
    torch.cuda.synchronize()
    assert (x.float() - x_ref.float()).abs().max() <= 2 ** -5  # one bf16 ulp at |x| < 8 (summation order)
    assert ((y.float() - y_ref).norm() / y_ref.norm()).item() < 6e-3


def test_qkv_finalize_matches_unfused_rope_and_cache_write():
    from skyrl_b200.ops import attention as attn_ops
    from skyrl_b200.ops import elementwise as ew

    torch.manual_seed(3)
    T, nq, nkv, D, P = 50, 12, 2, 128, 3
    W = (nq + 2 * nkv) * D
    part = torch.randn(P, T, W, device="cuda")
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    table = ew.build_rope_table(512, D, 1e6, "cuda")
    slots = torch.randperm(64 * 16, device="cuda")[:T].to(torch.int32)
    slots[5] = -1
    kc = torch.zeros(64, 16, nkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc)
    qkv = torch.empty(T, W, device="cuda", dtype=torch.bfloat16)
    ew.qkv_finalize(part, P, pos, table, qkv, kc, vc, slots, nq, nkv, D)
    ref = part.sum(0).to(torch.bfloat16)
    ref = ew.rope_(ref, pos, table, nq + nkv, D)
    attn_ops.kv_cache_write(ref, kc2, vc2, slots, nq, nkv, D)
    torch.cuda.synchronize()
    assert (qkv.float() - ref.float()).abs().max() <= 0.0625  # summation order may move a value by one bf16 ulp
    assert ((qkv.float() - ref.float()).norm() / ref.float().norm()).item() < 3e-3
    assert ((kc.float() - kc2.float()).norm() / kc2.float().norm()).item() < 3e-3
    assert ((vc.float() - vc2.float()).norm() / vc2.float().norm()).item() < 3e-3
    assert kc.view(-1, nkv * D)[slots[6].item()].abs().sum() > 0
