"""Grouped per-expert GEMM: layout plan (CPU) and the tcgen05 kernel against a plain fp32 reference (GPU)."""
import pytest
import torch

from skyrl_b200.ops import grouped_gemm as gg


def _case(n, E, K, N, device, dtype, seed=0, skew=False):
    g = torch.Generator().manual_seed(seed)
    if skew:  # a few experts take most rows, several get none
        ids = torch.randint(0, max(1, E // 4), (n,), generator=g)
    else:
        ids = torch.randint(0, E, (n,), generator=g)
    rows = (torch.randn(n, K, generator=g) * 0.5).to(dtype)
    w = (torch.randn(E, N, K, generator=g) * 0.05).to(dtype)
    return ids.to(device), rows.to(device), w.to(device)


def _reference(ids, rows, w):
    out = torch.zeros(rows.shape[0], w.shape[1], dtype=torch.float32, device=rows.device)
    for e in range(w.shape[0]):
        m = ids == e
        if m.any():
            out[m] = rows[m].float() @ w[e].float().t()
    return out


def _run(ids, rows, w, with_grad=True):
    E = w.shape[0]
    plan = gg.plan_groups(ids, E)
    rows = rows.clone().requires_grad_(with_grad)
    w = w.clone().requires_grad_(with_grad)
    x = torch.zeros((plan.m_cap, rows.shape[1]), device=rows.device, dtype=rows.dtype).index_copy(0, plan.dst_row, rows[plan.order])
    y_pad = gg.grouped_linear(x, w, plan)
    y_sorted = y_pad[plan.dst_row]
    y = torch.empty_like(y_sorted).index_copy(0, plan.order, y_sorted)  # back to the caller's order
    return plan, rows, w, y


def test_plan_layout_cpu():
    ids = torch.tensor([3, 0, 3, 3, 1, 0, 3])
    plan = gg.plan_groups(ids, 5)
    assert plan.k_off.tolist() == [0, 128, 256, 256, 384, 384]
    assert plan.m_cap % 128 == 0 and plan.m_cap >= 384
    te = plan.tile_expert.tolist()
    assert te[:3] == [0, 1, 3] and all(t == -1 for t in te[3:])
    # sorted entries land in their expert's range, in stable order
    assert plan.order.tolist() == [1, 5, 4, 0, 2, 3, 6]
    assert plan.dst_row.tolist() == [0, 1, 128, 256, 257, 258, 259]


def test_grouped_linear_cpu_matches_per_expert_reference():
    ids, rows, w = _case(300, 6, 32, 48, "cpu", torch.float32, skew=True)
    plan, rows_g, w_g, y = _run(ids, rows, w)
    ref_rows = rows.clone().requires_grad_()
    ref_w = w.clone().requires_grad_()
    ref = torch.zeros_like(y)
    for e in range(6):
        m = ids == e
        if m.any():
            ref[m] = ref_rows[m] @ ref_w[e].t()
    assert torch.allclose(y, ref, atol=1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    ref.backward(gy)
    assert torch.allclose(rows_g.grad, ref_rows.grad, atol=1e-5)
    assert torch.allclose(w_g.grad, ref_w.grad, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("n,E,K,N,skew", [(4096, 8, 512, 768, False), (1000, 16, 256, 320, True), (20000, 32, 1024, 1536, False),
                                          (64, 64, 128, 256, False)])
def test_grouped_kernel_forward_backward(n, E, K, N, skew):
    ids, rows, w = _case(n, E, K, N, "cuda", torch.bfloat16, seed=n, skew=skew)
    plan, rows_g, w_g, y = _run(ids, rows, w)
    ref = _reference(ids, rows, w)
    err = (y.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-6)
    assert err < 2e-2, float(err)
    gy = (torch.randn(n, N, device="cuda") * 0.5).to(torch.bfloat16)
    y.backward(gy)
    # fp32 references of both gradients
    dx_ref = torch.zeros(n, K, device="cuda")
    dw_ref = torch.zeros(E, N, K, device="cuda")
    for e in range(E):
        m = ids == e
        if m.any():
            dx_ref[m] = gy[m].float() @ w[e].float()
            dw_ref[e] = gy[m].float().t() @ rows[m].float()
    e1 = (rows_g.grad.float() - dx_ref).abs().max() / dx_ref.abs().max().clamp_min(1e-6)
    e2 = (w_g.grad.float() - dw_ref).abs().max() / dw_ref.abs().max().clamp_min(1e-6)
    assert e1 < 2e-2 and e2 < 2e-2, (float(e1), float(e2))


@pytest.mark.gpu
def test_grouped_weight_gradient_accumulates_into_main_grad():
    n, E, K, N = 3000, 8, 256, 512
    ids, rows, w = _case(n, E, K, N, "cuda", torch.bfloat16, seed=5, skew=True)
    plan = gg.plan_groups(ids, E)
    x = torch.zeros((plan.m_cap, K), device="cuda", dtype=torch.bfloat16).index_copy(0, plan.dst_row, rows[plan.order])
    w = w.clone().requires_grad_()
    w.main_grad = torch.full((E, N, K), 0.25, device="cuda", dtype=torch.float32)
    y = gg.grouped_linear(x, w, plan)
    gy_pad = torch.zeros_like(y)
    gy = (torch.randn(n, N, device="cuda") * 0.5).to(torch.bfloat16)
    gy_pad.index_copy_(0, plan.dst_row, gy[plan.order])
    y.backward(gy_pad)
    assert w.grad is None
    for e in range(E):
        m = ids == e
        ref = 0.25 + (gy[m].float().t() @ rows[m].float() if m.any() else 0.0)
        err = (w.main_grad[e] - ref).abs().max() / (ref.abs().max() if m.any() else 1.0)
        assert err < 2e-2, (e, float(err))


def _moe_reference(h, rt, wgu, wd, k):
    """Plain fp32 mixture-of-experts FFN: softmax router, top-k, renormalised weights, per-expert SwiGLU FFN."""
    T, H = h.shape
    E, F2, _ = wgu.shape
    F = F2 // 2
    probs = torch.softmax(h.float() @ rt.float().t(), -1)
    w, idx = torch.topk(probs, k, -1)
    w = w / w.sum(-1, keepdim=True)
    out = torch.zeros(T, H, dtype=torch.float32, device=h.device)
    for e in range(E):
        t, s = torch.nonzero(idx == e, as_tuple=True)
        if t.numel() == 0:
            continue
        gu = h[t].float() @ wgu[e].float().t()
        act = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
        out.index_add_(0, t, (act @ wd[e].float().t()) * w[t, s][:, None])
    return out


def test_moe_layer_cpu_matches_reference_with_gradients():
    from skyrl_b200.models.moe import moe_ffn

    g = torch.Generator().manual_seed(3)
    T, H, E, F, k = 50, 32, 6, 24, 2
    h = torch.randn(T, H, generator=g).requires_grad_()
    rt = torch.randn(E, H, generator=g).requires_grad_()
    wgu = (torch.randn(E, 2 * F, H, generator=g) * 0.2).requires_grad_()
    wd = (torch.randn(E, H, F, generator=g) * 0.2).requires_grad_()
    out = moe_ffn(h, rt, wgu, wd, k, True)
    ref_in = [t.detach().clone().requires_grad_() for t in (h, rt, wgu, wd)]
    ref = _moe_reference(*ref_in, k)
    assert torch.allclose(out, ref, atol=1e-4), float((out - ref).abs().max())
    gy = torch.randn(T, H, generator=g)
    out.backward(gy)
    ref.backward(gy)
    for a, b, name in zip((h, rt, wgu, wd), ref_in, ("h", "router", "wgu", "wd")):
        assert torch.allclose(a.grad, b.grad, atol=2e-4), (name, float((a.grad - b.grad).abs().max()))


@pytest.mark.gpu
def test_moe_layer_gpu_matches_fp32_reference():
    from skyrl_b200.models.moe import moe_ffn

    torch.manual_seed(0)
    T, H, E, F, k = 1500, 512, 16, 256, 4
    h = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    rt = (torch.randn(E, H, device="cuda") * 0.1).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    wd = (torch.randn(E, H, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    out = moe_ffn(h, rt, wgu, wd, k, True)
    ref_in = [t.detach().clone().float().requires_grad_() for t in (h, wgu, wd)]
    ref = _moe_reference(ref_in[0], rt, ref_in[1], ref_in[2], k)
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 3e-2, float(err)
    gy = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16)
    out.backward(gy)
    ref.backward(gy.float())
    for a, b, name in zip((h, wgu, wd), ref_in, ("h", "wgu", "wd")):
        e = (a.grad.float() - b.grad).abs().max() / b.grad.abs().max().clamp_min(1e-6)
        assert e < 5e-2, (name, float(e))


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,norm", [(1000, 128, 8, True), (333, 60, 4, False), (64, 8, 2, True), (500, 256, 1, True)])
def test_router_kernel_matches_torch(T, E, k, norm):
    from skyrl_b200.models.moe import _RouteFn

    torch.manual_seed(E + k)
    logits = (torch.randn(T, E, device="cuda") * 2.0).requires_grad_()
    w, idx = _RouteFn.apply(logits, k, norm)
    ref_l = logits.detach().clone().requires_grad_()
    probs = torch.softmax(ref_l, -1)
    wr, ir = torch.topk(probs, k, -1)
    if norm:
        wr = wr / wr.sum(-1, keepdim=True)
    assert torch.equal(idx.long().sort(-1).values, ir.sort(-1).values)
    order = idx.long().argsort(-1)
    order_r = ir.argsort(-1)
    assert torch.allclose(w.gather(-1, order), wr.gather(-1, order_r), atol=1e-5, rtol=1e-4)
    g = torch.randn(T, k, device="cuda")
    # same gradient per selected expert on both sides (the two orders of the k slots may differ)
    g_ref = torch.zeros(T, E, device="cuda").scatter(-1, idx.long(), g).gather(-1, ir)
    w.backward(g)
    wr.backward(g_ref)
    assert torch.allclose(logits.grad, ref_l.grad, atol=2e-5, rtol=1e-3), float((logits.grad - ref_l.grad).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("n,E,k", [(7, 5, 1), (4096, 8, 2), (65536, 128, 8), (1000, 300, 4), (33, 1024, 1)])
def test_plan_kernel_matches_reference_plan(n, E, k):
    g = torch.Generator().manual_seed(n + E)
    ids = torch.randint(0, E, (n,), generator=g)
    ref = gg.plan_groups(ids, E, k)  # CPU path
    for dt in (torch.int64, torch.int32):
        got = gg.plan_groups(ids.to("cuda", dt), E, k)
        assert got.m_cap == ref.m_cap
        assert torch.equal(got.k_off.cpu(), ref.k_off)
        assert torch.equal(got.tile_expert.cpu(), ref.tile_expert)
        assert torch.equal(got.slot_row.cpu(), ref.slot_row)
        assert torch.equal(got.row_src.cpu(), ref.row_src)
        assert torch.equal(got.order.cpu(), ref.order) and torch.equal(got.dst_row.cpu(), ref.dst_row)
