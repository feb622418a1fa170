"""tcgen05 GEMM against an fp32 PyTorch reference, all operand layouts and ragged shapes."""
import pytest
import torch

from skyrl_b200.ops import _lib, gemm

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 1536, 1536), (1000, 2048, 1536), (77, 136, 72), (4096, 8960, 1536), (130, 152064 // 8, 512)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_nt(M, N, K, bn):
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    y = gemm.gemm_nt(x, w, b, bn_hint=bn)
    ref = x.float() @ w.float().t() + b.float()
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    assert _rel_err(y, ref) < 6e-3


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nn(M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    y = gemm.gemm_nn(a, b)
    ref = a.float() @ b.float()
    assert _lib.status_read_clear() == 0
    assert _rel_err(y, ref) < 6e-3


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tn(M, N, K):
    M = (M + 7) // 8 * 8  # the stored [K, M] operand needs 16-byte aligned rows
    torch.manual_seed(2)
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float().t() @ b.float()
    y = gemm.gemm_tn(a, b, out_dtype=torch.float32)
    assert _lib.status_read_clear() == 0
    assert _rel_err(y, ref) < 1e-3
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    gemm.gemm_tn(a, b, out=acc, accumulate=True)
    assert _rel_err(acc, ref + 1.0) < 1e-3


def test_linear_autograd():
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gemm.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(x.grad, xr.grad) < 6e-3
    assert _rel_err(w.grad, wr.grad) < 6e-3
    assert _rel_err(b.grad, br.grad) < 6e-3


# ------------------------------------------------------------------ tensor-parallel modes, ranks emulated on one GPU
def _tp_call(A, B, C, M, N, K, b_mn, out_mode, gather, scatter, peers, outs, n_ranks, my_rank, rpr, slot_stride, flags, bn=0):
    import ctypes

    from skyrl_b200.ops import _lib
    from skyrl_b200.parallel import tensor_parallel as tpm

    lib = tpm._k()
    pa = (ctypes.c_void_p * n_ranks)(*peers) if peers else None
    oa = (ctypes.c_void_p * n_ranks)(*outs) if outs else None
    code = lib.sb_gemm_tp(A.data_ptr(), B.data_ptr(), None if C is None else C.data_ptr(), None, M, N, K, A.stride(0),
                          B.stride(0), N, int(b_mn), out_mode, gather, scatter, pa, oa, n_ranks, my_rank, rpr, slot_stride,
                          None if flags is None else flags.data_ptr(), bn, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_tp")


@pytest.mark.parametrize("n_ranks,rpr,N,K,b_mn", [(2, 256, 384, 512, False), (4, 128, 1024, 1536, False), (2, 128, 256, 320, True)])
def test_gemm_gather_mode_matches_full_product(n_ranks, rpr, N, K, b_mn):
    """All-gather fused into the GEMM: every 'rank' is a separate local buffer here, launches run one after another
    (the kernel only waits on flags that its own copy warps set)."""
    from skyrl_b200.ops import _lib

    torch.manual_seed(0)
    M = n_ranks * rpr
    shards = [(torch.randn(rpr, K, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(n_ranks)]
    W = (torch.randn(K, N, device="cuda") * 0.05).to(torch.bfloat16) if b_mn else \
        (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    x_all = torch.cat(shards, 0)
    ref = x_all.float() @ (W.float() if b_mn else W.float().t())
    flags = torch.zeros(M // 128 + 1, dtype=torch.int32, device="cuda")
    for me in range(n_ranks):
        a_full = torch.full((M, K), float("nan"), device="cuda", dtype=torch.bfloat16)
        a_full[me * rpr : (me + 1) * rpr] = shards[me]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        _tp_call(a_full, W, out, M, N, K, b_mn, 0, 1, 0, [s.data_ptr() for s in shards], None, n_ranks, me, rpr, 0, flags)
        torch.cuda.synchronize()
        assert _lib.status_read_clear() == 0
        assert torch.equal(a_full, x_all)  # the gathered operand is left behind for the backward pass
        assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2


@pytest.mark.parametrize("all_ranks", [False, True])
def test_gemm_scatter_mode_slots_sum_to_product(all_ranks):
    from skyrl_b200.ops import _lib

    torch.manual_seed(1)
    n_ranks, rpr, N, Kloc = 4, 96, 512, 256
    M = n_ranks * rpr
    xs = [(torch.randn(M, Kloc, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(n_ranks)]
    ws = [(torch.randn(N, Kloc, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(n_ranks)]
    ref = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    rows = M if all_ranks else rpr
    dests = [torch.full((n_ranks, rows, N), float("nan"), device="cuda") for _ in range(n_ranks)]
    for me in range(n_ranks):
        _tp_call(xs[me], ws[me], None, M, N, Kloc, False, 1, 0, 2 if all_ranks else 1, None, [d.data_ptr() for d in dests],
                 n_ranks, me, M if all_ranks else rpr, rows * N, None)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    for d in range(n_ranks):
        got = dests[d].sum(0)
        want = ref if all_ranks else ref[d * rpr : (d + 1) * rpr]
        assert torch.isfinite(got).all()
        assert ((got - want).norm() / want.norm()).item() < 2e-3


def _sp_call(A, B, C, M, N, K, mode, peers, n_ranks, my_rank, rpr, seg_start=None, seg_w=None, cpr=0, src_ld=0, flags=None,
             ldc=None, bias=None):
    import ctypes

    from skyrl_b200.ops import _lib
    from skyrl_b200.parallel import ulysses

    lib = ulysses._k()
    pa = (ctypes.c_void_p * n_ranks)(*peers)
    ss = (ctypes.c_int * 3)(*seg_start) if seg_start else None
    sw = (ctypes.c_int * 3)(*seg_w) if seg_w else None
    code = lib.sb_gemm_sp(A.data_ptr(), B.data_ptr(), None if C is None else C.data_ptr(),
                          None if bias is None else bias.data_ptr(), M, N, K, A.stride(0), B.stride(0),
                          ldc if ldc is not None else N, mode, pa, n_ranks, my_rank, rpr, ss, sw, cpr, src_ld,
                          None if flags is None else flags.data_ptr(), 0, _lib.stream_ptr())
    _lib.check(code, "sb_gemm_sp")


def test_gemm_column_scatter_matches_all_to_all_layout():
    """QKV projection whose epilogue performs the sequence-to-head exchange (ranks emulated by local buffers)."""
    from skyrl_b200.ops import _lib

    torch.manual_seed(2)
    sp, R, K = 2, 200, 512
    widths = [512, 256, 256]  # q | k | v
    N = sum(widths)
    per = [w // sp for w in widths]
    local = sum(per)
    starts = [0, 512, 768]
    W = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device="cuda").to(torch.bfloat16)
    xs = [(torch.randn(R, K, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(sp)]
    dests = [torch.full((sp * R, local), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(sp)]
    for me in range(sp):
        _sp_call(xs[me], W, None, R, N, K, 1, [d.data_ptr() for d in dests], sp, me, R, starts, per, ldc=local, bias=b)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    for d in range(sp):
        for src in range(sp):
            full = xs[src].float() @ W.float().t() + b.float()
            want = torch.cat([full[:, s + d * p : s + (d + 1) * p] for s, p in zip(starts, per)], 1)
            got = dests[d][src * R : (src + 1) * R].float()
            assert torch.isfinite(got).all()
            assert ((got - want).norm() / want.norm()).item() < 1e-2


def test_gemm_column_gather_matches_head_to_seq_then_project():
    from skyrl_b200.ops import _lib

    torch.manual_seed(3)
    sp, R, cpr, H = 4, 150, 128, 384
    K = sp * cpr
    atts = [(torch.randn(sp * R, cpr, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(sp)]  # rank r: all tokens, its heads
    Wo = (torch.randn(H, K, device="cuda") * 0.05).to(torch.bfloat16)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    for me in range(sp):
        a_full = torch.full((R, K), float("nan"), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(R, H, device="cuda", dtype=torch.bfloat16)
        _sp_call(a_full, Wo, out, R, H, K, 2, [a.data_ptr() for a in atts], sp, me, R, cpr=cpr, src_ld=cpr, flags=flags)
        torch.cuda.synchronize()
        assert _lib.status_read_clear() == 0
        want_a = torch.cat([atts[r][me * R : (me + 1) * R] for r in range(sp)], 1)
        assert torch.equal(a_full, want_a)
        ref = want_a.float() @ Wo.float().t()
        assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2


def test_gemm_indexed_dispatch_and_combine():
    """Expert GEMMs with token dispatch (indexed row gather from 'peer' buffers) and combine (indexed row scatter)."""
    import ctypes

    from skyrl_b200.ops import _lib
    from skyrl_b200.parallel import expert_parallel as epm

    torch.manual_seed(4)
    n_ranks, T, H, F2, n = 3, 40, 256, 512, 150
    hid = [(torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(n_ranks)]
    W1 = (torch.randn(F2, H, device="cuda") * 0.05).to(torch.bfloat16)
    src_rank = torch.randint(0, n_ranks, (n,), device="cuda", dtype=torch.int32)
    src_row = torch.randint(0, T, (n,), device="cuda", dtype=torch.int32)
    a_full = torch.full((n, H), float("nan"), device="cuda", dtype=torch.bfloat16)
    out = torch.empty(n, F2, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    peers = (ctypes.c_void_p * n_ranks)(*[h.data_ptr() for h in hid])
    lib = epm._k()
    _lib.check(lib.sb_gemm_ep(a_full.data_ptr(), W1.data_ptr(), out.data_ptr(), n, F2, H, H, H, F2, 0, 1, peers, n_ranks, 1,
                              src_rank.data_ptr(), src_row.data_ptr(), H, flags.data_ptr(), 0, _lib.stream_ptr()), "dispatch")
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    want_rows = torch.stack(hid)[src_rank.long(), src_row.long()]
    assert torch.equal(a_full, want_rows)
    ref = want_rows.float() @ W1.float().t()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
    # combine: rows go to (rank, slot) of zero-initialised buffers; slots are unique per destination
    W2 = (torch.randn(H, F2, device="cuda") * 0.05).to(torch.bfloat16)
    x = (torch.randn(n, F2, device="cuda") * 0.5).to(torch.bfloat16)
    dst_rank = torch.randint(0, n_ranks, (n,), device="cuda", dtype=torch.int32)
    dst_row = torch.empty(n, device="cuda", dtype=torch.int32)
    for d in range(n_ranks):
        sel = (dst_rank == d).nonzero(as_tuple=True)[0]
        dst_row[sel] = torch.randperm(200, device="cuda")[: sel.numel()].to(torch.int32)
    bufs = [torch.zeros(200, H, device="cuda", dtype=torch.bfloat16) for _ in range(n_ranks)]
    pc = (ctypes.c_void_p * n_ranks)(*[b.data_ptr() for b in bufs])
    _lib.check(lib.sb_gemm_ep(x.data_ptr(), W2.data_ptr(), None, n, H, F2, F2, F2, H, 0, 2, pc, n_ranks, 0,
                              dst_rank.data_ptr(), dst_row.data_ptr(), 0, None, 0, _lib.stream_ptr()), "combine")
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    y = x.float() @ W2.float().t()
    for d in range(n_ranks):
        sel = (dst_rank == d).nonzero(as_tuple=True)[0]
        got = bufs[d][dst_row[sel].long()].float()
        assert ((got - y[sel]).norm() / y[sel].norm()).item() < 1e-2
        untouched = torch.ones(200, dtype=torch.bool, device="cuda")
        untouched[dst_row[sel].long()] = False
        assert bufs[d][untouched].abs().sum() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (300, 384, 200), (1000, 520, 1536), (128, 256, 320)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("bn", [256, 128])
def test_gemm_cta_pair_kernel(M, N, K, a_mn, b_mn, bn):
    from skyrl_b200.ops import _lib, gemm

    torch.manual_seed(0)
    M8, N8 = (M + 7) // 8 * 8, (N + 7) // 8 * 8
    A = (torch.randn(K, M8, device="cuda") * 0.5).to(torch.bfloat16) if a_mn else (torch.randn(M8, K + (-K) % 8, device="cuda") * 0.5).to(torch.bfloat16)
    Kp = K if a_mn else A.shape[1]
    B = (torch.randn(Kp, N8, device="cuda") * 0.1).to(torch.bfloat16) if b_mn else (torch.randn(N8, Kp, device="cuda") * 0.1).to(torch.bfloat16)
    Af = A.float().t() if a_mn else A.float()
    Bf = B.float() if b_mn else B.float().t()
    ref = Af @ Bf
    out = torch.full((M8, N8), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.gemm_2cta(A, B, out, a_mn=a_mn, b_mn=b_mn, bn=bn)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0
    assert torch.isfinite(out.float()).all()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
    acc = torch.ones((M8, N8), device="cuda", dtype=torch.float32)
    gemm.gemm_2cta(A, B, acc, a_mn=a_mn, b_mn=b_mn, accumulate=True, bn=bn)
    torch.cuda.synchronize()
    assert ((acc - 1 - ref).norm() / ref.norm()).item() < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("M,H,F", [(1024, 512, 1280), (2304, 1536, 8960), (777 + 256, 256, 384)])
def test_fused_swiglu_mlp_matches_unfused(M, H, F):
    """SwiGLU fused into the gate/up GEMM epilogue (forward) and into the down-projection input gradient (backward)
    against the plain composition and an fp32 reference."""
    import os

    from skyrl_b200.ops import elementwise as ew

    torch.manual_seed(M)
    x = (torch.randn(M, H, device="cuda") * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(2 * F, H, device="cuda") * 0.05).to(torch.bfloat16)
    wd = (torch.randn(H, F, device="cuda") * 0.05).to(torch.bfloat16)
    gy = (torch.randn(M, H, device="cuda") * 0.5).to(torch.bfloat16)

    def run(fn):
        xs, a, b = x.clone().requires_grad_(), wgu.clone().requires_grad_(), wd.clone().requires_grad_()
        y = fn(xs, a, b)
        y.backward(gy)
        return y.detach().float(), xs.grad.float(), a.grad.float(), b.grad.float()

    assert gemm.mlp_fusable(x, wgu, wd)
    fused = run(gemm.swiglu_mlp)
    plain = run(lambda xs, a, b: gemm.linear(ew.swiglu(gemm.linear(xs, a)), b))

    def ref(xs, a, b):
        gu = xs.float() @ a.float().t()
        return (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ b.float().t()

    xs, a, b = x.float().requires_grad_(), wgu.float().requires_grad_(), wd.float().requires_grad_()
    yr = ref(xs, a, b)
    yr.backward(gy.float())
    refs = (yr.detach(), xs.grad, a.grad, b.grad)
    for name, f, p_, r in zip(("y", "dx", "dwgu", "dwd"), fused, plain, refs):
        scale = r.abs().max().clamp_min(1e-6)
        assert (f - r).abs().max() / scale < 3e-2, (name, float((f - r).abs().max() / scale))
        assert (f - p_).abs().max() / scale < 2e-2, (name, "vs unfused", float((f - p_).abs().max() / scale))
    # forward-only callers skip the gate/up store
    with torch.no_grad():
        y2 = gemm.swiglu_mlp(x, wgu, wd).float()
    assert torch.equal(y2, fused[0])
