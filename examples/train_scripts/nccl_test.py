"""Sanity check of the collective fabric before a run: all-reduce, all-gather and all-to-all across every rank, timed on
the device (CUDA events, max over ranks), with the bus bandwidth NCCL's own tests report.  On a machine without GPUs
it runs over gloo on the CPU and only checks the results.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_scripts/nccl_test.py --mib 256

Counterpart in the reference: examples/train_scripts/multi_node_nccl_test.py.
"""

import argparse
import time

import torch
import torch.distributed as dist

from skyrl_b200.parallel import dist as pdist


def timed(fn, iters: int, cuda: bool) -> float:
    """Seconds per call: device time between two events on the launching stream, max over ranks."""
    for _ in range(3):
        fn()
    if cuda:
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        e1.synchronize()
        dt = e0.elapsed_time(e1) / 1e3 / iters
    else:
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        dt = (time.perf_counter() - t0) / iters
    t = torch.tensor([dt], dtype=torch.float64, device="cuda" if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=float, default=64.0, help="payload per rank")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    env = pdist.init_distributed()
    cuda = env.device.type == "cuda"
    W, r = env.world_size, env.rank
    n = max(W, int(a.mib * 2**20 / 4) // W * W)
    x = torch.full((n,), float(r + 1), device=env.device)
    # correctness first
    y = x.clone()
    dist.all_reduce(y)
    assert torch.allclose(y, torch.full_like(y, W * (W + 1) / 2)), "all_reduce returned a wrong sum"
    parts = [torch.empty(n // W, device=env.device) for _ in range(W)]
    dist.all_gather(parts, x[: n // W])
    assert all(float(p[0]) == i + 1 for i, p in enumerate(parts)), "all_gather mixed up the ranks"
    if cuda or W == 1:
        z = torch.empty_like(x)
        dist.all_to_all_single(z, x)
        assert all(float(z[i * (n // W)]) == i + 1 for i in range(W)), "all_to_all mixed up the ranks"
    size = n * 4
    rows = []
    t = timed(lambda: dist.all_reduce(y), a.iters, cuda)
    rows.append(("all_reduce", t, size / t * 2 * (W - 1) / max(1, W)))
    t = timed(lambda: dist.all_gather(parts, x[: n // W]), a.iters, cuda)
    rows.append(("all_gather", t, size / t * (W - 1) / max(1, W)))
    if cuda or W == 1:
        t = timed(lambda: dist.all_to_all_single(z, x), a.iters, cuda)
        rows.append(("all_to_all", t, size / t * (W - 1) / max(1, W)))
    if env.is_main:
        for name, t, bus in rows:
            print(f"{name:>11}: {size / 2**20:8.1f} MiB  {t * 1e3:9.3f} ms  bus {bus / 1e9:8.2f} GB/s  ({W} ranks, "
                  f"{'device events' if cuda else 'host clock'})")
        print("NCCL_TEST_OK" if cuda else "GLOO_TEST_OK")
    pdist.shutdown()


if __name__ == "__main__":
    main()
