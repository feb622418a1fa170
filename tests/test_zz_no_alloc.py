"""The allocation-free LM-head entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need log-probabilities (a serving
loop that has frozen its memory pool, a host process that bans cudaMalloc after start-up).  For them the library
exports ``sb_lmhead_logprob_noalloc``, which keeps its scratch in a fixed array inside the library.  This test
checks it against the regular entry point (whose scratch the caller allocates) on two consecutive calls with
different inputs -- the second call sees the first call's leftovers in the shared scratch -- and checks that an
oversized request is refused rather than overrunning the array.
"""
import ctypes

import pytest
import torch

from skyrl_b200.ops import _lib, lm_head

pytestmark = pytest.mark.gpu

MAX_RECORDS = 262144


def _call_noalloc(lib, h, W, tgt, inv_temp):
    T, K = h.shape
    V = W.shape[0]
    lp = torch.empty(T, device="cuda", dtype=torch.float32)
    ent = torch.empty_like(lp)
    lse = torch.empty_like(lp)
    code = lib.sb_lmhead_logprob_noalloc(h.data_ptr(), W.data_ptr(), tgt.data_ptr(), T, V, K, h.stride(0), W.stride(0),
                                         inv_temp, lp.data_ptr(), ent.data_ptr(), lse.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    return code, lp, ent, lse


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib.kernels()
    vp, ci, cl, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.sb_lmhead_logprob_noalloc.argtypes = [vp, vp, vp, ci, ci, ci, cl, cl, cf, vp, vp, vp, vp]
    lib.sb_lmhead_logprob_noalloc.restype = ci
    for call, (T, V, K, temp) in enumerate([(700, 32000, 512, 1.0), (333, 151936, 1536, 0.7)]):
        torch.manual_seed(call)
        h = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
        W = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16)
        tgt = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        code, lp, ent, lse = _call_noalloc(lib, h, W, tgt, 1.0 / temp)
        assert code == 0
        ref_lp, ref_ent = lm_head.lm_head_logprobs(h, W, tgt, 1.0 / temp, with_entropy=True)
        torch.cuda.synchronize()
        assert _lib.status_read_clear() == 0
        # same kernels, same split layout: the two entry points agree to rounding
        assert torch.allclose(lp, ref_lp, atol=1e-5, rtol=1e-5), (call, (lp - ref_lp).abs().max())
        assert torch.allclose(ent, ref_ent, atol=1e-5, rtol=1e-5), (call, (ent - ref_ent).abs().max())
        z = (h.float() @ W.float().t()) / temp
        assert (lse - torch.logsumexp(z, -1)).abs().max() < 3e-2


def test_noalloc_rejects_requests_beyond_the_scratch():
    lib = _lib.kernels()
    vp, ci, cl, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.sb_lmhead_logprob_noalloc.argtypes = [vp, vp, vp, ci, ci, ci, cl, cl, cf, vp, vp, vp, vp]
    lib.sb_lmhead_logprob_noalloc.restype = ci
    lib.sb_lmhead_num_splits.argtypes = [ci, ci]
    T, V, K = 300000, 512, 64
    assert T * lib.sb_lmhead_num_splits(T, V) > MAX_RECORDS
    h = torch.zeros(T, K, device="cuda", dtype=torch.bfloat16)
    W = torch.zeros(V, K, device="cuda", dtype=torch.bfloat16)
    tgt = torch.zeros(T, device="cuda", dtype=torch.int32)
    code, *_ = _call_noalloc(lib, h, W, tgt, 1.0)
    assert code == 4  # SB_ERR_TOO_LARGE: refused, nothing launched
