"""Run under torchrun on CPU (gloo), world size 4: hybrid sharding (2 replicas x 2 shards) of the flat optimizer."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel.sharded_optimizer import ShardedAdamW  # noqa: E402


def main():
    env = pdist.init_distributed(backend="gloo", device="cpu")
    assert env.world_size == 4
    shard_g, replica_g = pdist.build_hsdp_groups(2, env)
    assert dist.get_world_size(shard_g) == 2 and dist.get_world_size(replica_g) == 2
    N = 256
    torch.manual_seed(0)
    p = torch.randn(N)
    ref = p.clone().requires_grad_()
    opt_ref = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    grads = torch.zeros(N)
    opt = ShardedAdamW(p, grads, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1e9, group=shard_g,
                       replica_group=replica_g, transport="nccl")
    assert opt.master.numel() == N // 2, "state must be sharded over the shard group only"
    for step in range(3):
        torch.manual_seed(10 * step + env.rank)
        g_local = torch.randn(N)
        grads.copy_(g_local)
        g_sum = g_local.clone()
        dist.all_reduce(g_sum)
        ref.grad = g_sum
        norm = opt.step()
        opt.zero_grad()
        opt_ref.step()
        err = ((p - ref.detach()).norm() / ref.detach().norm()).item()
        assert err < 1e-5, (step, err)
        assert abs(float(norm) - float(g_sum.norm())) < 1e-3 * float(g_sum.norm())
    # all four ranks hold identical parameters
    parts = [torch.empty_like(p) for _ in range(4)]
    dist.all_gather(parts, p)
    assert all(torch.equal(parts[0], x) for x in parts)
    dist.barrier()
    if env.rank == 0:
        print("HSDP_OK")
    pdist.shutdown()


if __name__ == "__main__":
    main()
