"""A device-side wait that runs out is acted upon: the fused optimizer publishes nothing and the worker raises.

The failure is made without faulting anything: a barrier is enqueued for an epoch that the (absent) second rank never
signals, with a 0.2 s limit; the kernel records a status code and returns, and the context stays usable.
"""
import ctypes

import pytest
import torch

from skyrl_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _peer_lib():
    from skyrl_b200.parallel import peer

    return peer._k()


def test_timed_out_barrier_blocks_the_parameter_push_and_is_reported():
    lib = _peer_lib()
    dev = torch.device("cuda:0")
    assert _lib.status_read_clear() == 0
    n = 4096
    master = torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    grad = torch.randn(n, device=dev)
    params = master.to(torch.bfloat16)
    before_master, before_params = master.clone(), params.clone()
    norm_pad = torch.tensor([float(grad.pow(2).sum()), 0, 0, 0, 0, 0, 0, 0], device=dev)
    norm, skipped = torch.zeros(1, device=dev), torch.zeros(1, device=dev, dtype=torch.int32)
    parr = (ctypes.c_void_p * 1)(params.data_ptr())

    def step():
        _lib.check(lib.sb_peer_adamw_push(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), parr, 1, 0, n,
                                          1e-2, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, norm_pad.data_ptr(), 1.0, 1.0,
                                          norm.data_ptr(), skipped.data_ptr(), _lib.stream_ptr()), "sb_peer_adamw_push")

    # two signal pads on this one GPU stand for two ranks; nothing ever writes "rank 1"'s flag into pad 0
    pad0 = torch.zeros(64, device=dev, dtype=torch.int32)
    pad1 = torch.zeros(64, device=dev, dtype=torch.int32)
    pads = (ctypes.c_void_p * 2)(pad0.data_ptr(), pad1.data_ptr())
    _lib.check(lib.sb_peer_barrier(pads, 0, 2, 0, 1, int(0.2e9), _lib.stream_ptr()), "sb_peer_barrier")
    step()
    torch.cuda.synchronize()
    assert int(skipped) == 2, "the update must be withheld once a wait has timed out"
    assert torch.equal(master, before_master) and torch.equal(params, before_params)
    assert torch.count_nonzero(m) == 0 and torch.count_nonzero(v) == 0

    # the worker turns the status word into an exception (and clears it)
    from types import SimpleNamespace

    from skyrl_b200.workers.worker import DeviceWaitError, ModelWorker

    w = ModelWorker.__new__(ModelWorker)
    w.env, w.role = SimpleNamespace(device=dev, rank=0), "policy"
    with pytest.raises(DeviceWaitError) as ei:
        w.check_device_status("optim_step")
    assert "0x901" in str(ei.value)  # barrier code 0x900 | the peer that never arrived
    w.check_device_status("optim_step")  # cleared: no second report

    # with a clean status word the same call updates the parameters
    step()
    torch.cuda.synchronize()
    assert int(skipped) == 0 and not torch.equal(master, before_master) and not torch.equal(params, before_params)
    assert _lib.status_read_clear() == 0
