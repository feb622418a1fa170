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
