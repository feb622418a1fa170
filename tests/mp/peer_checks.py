"""Run under torchrun with 2+ GPUs: peer-memory collectives against NCCL references."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.ops import _lib  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel.peer import PeerContext  # noqa: E402
from skyrl_b200.parallel.sharded_optimizer import ShardedAdamW  # noqa: E402


def main():
    env = pdist.init_distributed()
    dev, W, r = env.device, env.world_size, env.rank
    ctx = PeerContext(dev, wait_seconds=5.0)
    for _ in range(3):
        ctx.barrier(0)
    torch.cuda.synchronize()
    assert _lib.status_read_clear() == 0

    # all-reduce
    n = 1 << 16
    buf = ctx.alloc(n, torch.bfloat16)
    torch.manual_seed(r)
    x = torch.randn(n, device=dev).to(torch.bfloat16)
    buf.local.copy_(x)
    out = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ctx.all_reduce_bf16(buf, out)
    ref = x.float().clone()
    dist.all_reduce(ref)
    assert (out.float() - ref).abs().max() < 0.1, (out.float() - ref).abs().max()

    # fused optimizer (peer) == NCCL optimizer
    N = 8192 * 16
    torch.manual_seed(0)
    p0 = torch.randn(N).to(torch.bfloat16)
    params_s, grads_s = ctx.alloc(N, torch.bfloat16), ctx.alloc(N, torch.float32)
    params_s.local.copy_(p0.to(dev))
    params_n = p0.to(dev).clone()
    grads_n = torch.zeros(N, device=dev)
    opt_p = ShardedAdamW(params_s.local, grads_s.local, lr=1e-2, max_grad_norm=1.0, peer_ctx=ctx, params_symm=params_s,
                         grads_symm=grads_s)
    opt_n = ShardedAdamW(params_n, grads_n, lr=1e-2, max_grad_norm=1.0, transport="nccl")
    assert opt_p.transport == "peer" and opt_n.transport == "nccl"
    for step in range(3):
        torch.manual_seed(100 * step + r)
        g = torch.randn(N, device=dev)
        grads_s.local.copy_(g)
        grads_n.copy_(g)
        n1 = opt_p.step()
        n2 = opt_n.step()
        opt_p.zero_grad()
        opt_n.zero_grad()
        torch.cuda.synchronize()
        assert abs(float(n1) - float(n2)) / float(n2) < 1e-4, (float(n1), float(n2))
        # same math, different summation order of the norm partials: allow one bf16 ulp
        assert torch.allclose(params_s.local.float(), params_n.float(), rtol=1.6e-2, atol=1e-3), \
            (params_s.local.float() - params_n.float()).abs().max()
    # every rank ends with identical parameters
    chk = params_s.local.float().sum()
    lst = [torch.zeros_like(chk) for _ in range(W)]
    dist.all_gather(lst, chk)
    assert all(torch.equal(lst[0], t) for t in lst)

    # push with cast into a peer-visible "engine" buffer
    eng = ctx.alloc(N, torch.bfloat16)
    src = torch.randn(N // W, device=dev)
    ctx.push_bf16(src, eng.ptrs, dst_offset=r * (N // W))
    ctx.barrier(4)
    torch.cuda.synchronize()
    assert torch.equal(eng.local[r * (N // W):(r + 1) * (N // W)], src.to(torch.bfloat16))
    assert _lib.status_read_clear() == 0

    # a barrier nobody else joins runs out after its bound and reports a status instead of hanging
    if os.environ.get("SB_TEST_BARRIER_TIMEOUT", "1") == "1":
        dist.barrier()
        short = PeerContext.__new__(PeerContext)
        short.__dict__.update(ctx.__dict__)
        short.wait_ns = int(0.2e9)
        if r == 0:
            short._epoch = list(ctx._epoch)
            short._epoch[5] = 1000  # peers never reach this epoch on channel 5
            short.barrier(5)
            torch.cuda.synchronize()
            st = _lib.status_read_clear()
            assert (st & 0xF00) == 0x900, hex(st)
        dist.barrier()
    dist.barrier()
    if r == 0:
        print("PEER_CHECKS_OK world", W, flush=True)
    ctx.close()
    pdist.shutdown()


if __name__ == "__main__":
    main()
