"""Run under torchrun on CPU (gloo), any world size >= 2:  python cp_check.py

Context parallelism by key/value all-gather: the sharded model's log-probs equal the plain model's, and the weight
gradients summed over the ranks equal the plain model's gradients -- also when the degree does not divide the number
of key/value heads (which Ulysses cannot do) and when a rank's slice starts in the middle of a sequence.
"""
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.models.decoder import PRESETS, CausalLM  # noqa: E402
from skyrl_b200.models.tp_decoder import ContextParallelCausalLM, pad_packed_for_tp  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel import tensor_parallel as tpm  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    env = pdist.init_distributed(backend="gloo", device="cpu")
    W = env.world_size
    cp = tpm.TPGroup(None)
    a = dataclasses.replace(PRESETS["tiny-llama"], num_kv_heads=2, num_heads=4, attention_bias=True)
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=5)
    m = ContextParallelCausalLM(a, cp, device="cpu", dtype=torch.float32, seed=5)
    for lens in ([30, 61, 200], [517], [3, 3, 3, 700, 9]):
        for mm in (full, m):
            for _, prm in mm.named_flat_views():
                prm.grad = None
        ids = torch.randint(4, a.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(2)).int()
        pos = torch.cat([torch.arange(n) for n in lens]).int()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0))).int()
        ids_p, pos_p, cu_p, T = pad_packed_for_tp(ids, pos, cu, W)
        tgt = torch.roll(ids_p.long(), -1)
        wts = torch.zeros(ids_p.numel())
        wts[:T] = torch.rand(T, generator=torch.Generator().manual_seed(3))
        lp, _ = m.token_logprobs_full(m(ids_p, pos_p, cu_p, max(lens)), tgt)
        (lp * wts).sum().backward()
        lpf, _ = full.token_logprobs(full(ids_p, pos_p, cu_p, max(lens)), tgt)
        (lpf * wts).sum().backward()
        assert rel(lp[:T], lpf[:T]) < 1e-4, (lens, rel(lp[:T], lpf[:T]))
        for name, prm in m.named_flat_views():
            g = prm.grad.clone() if prm.grad is not None else torch.zeros_like(prm)
            dist.all_reduce(g)
            assert rel(g, full.p(name).grad) < 2e-3, (lens, name, rel(g, full.p(name).grad))
    dist.barrier()
    if env.rank == 0:
        print(f"CP_MODEL_OK world={W} kv_heads={a.num_kv_heads}")
    pdist.shutdown()


if __name__ == "__main__":
    main()
