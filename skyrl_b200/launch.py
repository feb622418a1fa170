"""Process launcher: one worker process per GPU on this node, with the environment the workers expect.

    python -m skyrl_b200.launch --nproc-per-node 8 -m skyrl_b200.entrypoints.main_base key=value ...
    python -m skyrl_b200.launch --nproc-per-node 2 path/to/script.py args...

This is the single-node counterpart of what the reference does with Ray: runtime environment export
(skyrl/train/utils/utils.py:682-845), placement of rank *i* on physical GPU *i* (:948-1033), actor-group start-up with
master address/port discovery (skyrl/backends/skyrl_train/workers/worker.py:591-828) and NUMA pinning of each worker
to the node nearest its GPU (worker.py:180-287).  Differences by design: there is no scheduler and no object store;
ranks are plain OS processes that rendezvous over 127.0.0.1, and the launcher doubles as the failure detector: when
any rank exits non-zero (or is killed) the remaining ranks receive SIGTERM, then SIGKILL after a grace period, and the
launcher's exit code is the first failing rank's.
"""

from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def peer_access_supported(n: int) -> bool:
    """True when every visible GPU pair reports peer access (decides whether NCCL P2P may be used)."""
    try:
        import torch

        if not torch.cuda.is_available() or torch.cuda.device_count() < n:
            return False
        return all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j)
    except Exception:
        return False


def gpu_numa_node(index: int) -> Optional[int]:
    """NUMA node of GPU ``index`` from sysfs (``None`` when it cannot be determined)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        path = f"/sys/bus/pci/devices/{bus[-12:].lower()}/numa_node"
        with open(path) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def numa_cpus(node: int) -> List[int]:
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
    except OSError:
        return []
    cpus: List[int] = []
    for part in spec.split(","):
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        elif part:
            cpus.append(int(part))
    return cpus


def prepare_runtime_environment(nproc: int, base: Optional[Dict[str, str]] = None, check_peers: bool = True) -> Dict[str, str]:
    """Environment shared by every rank (the launcher adds the per-rank variables)."""
    env = dict(os.environ if base is None else base)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("MASTER_PORT", str(_free_port()))
    env.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 8) // max(nproc, 1))))
    env.setdefault("TOKENIZERS_PARALLELISM", "false")
    env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
    env.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
    if check_peers and nproc > 1 and not peer_access_supported(nproc):
        # without peer access neither NCCL P2P nor the peer-memory kernels can be used
        env.setdefault("NCCL_P2P_DISABLE", "1")
        env.setdefault("NCCL_SHM_DISABLE", "1")
        env.setdefault("SKYRL_B200_DISABLE_PEER_KERNELS", "1")
    return env


class WorkerGroup:
    """Spawns ``nproc`` ranks of one command and supervises them."""

    def __init__(self, cmd: List[str], nproc: int, env: Optional[Dict[str, str]] = None, numa_pin: bool = True,
                 node_rank: int = 0, nnodes: int = 1, grace_s: float = 10.0):
        self.cmd, self.nproc, self.grace_s = cmd, nproc, grace_s
        self.node_rank, self.nnodes = node_rank, nnodes
        self.env = prepare_runtime_environment(nproc, env)
        self.numa_pin = numa_pin
        self.procs: List[subprocess.Popen] = []

    def start(self) -> "WorkerGroup":
        world = self.nproc * self.nnodes
        for local in range(self.nproc):
            e = dict(self.env)
            e.update({"RANK": str(self.node_rank * self.nproc + local), "LOCAL_RANK": str(local), "WORLD_SIZE": str(world),
                      "LOCAL_WORLD_SIZE": str(self.nproc), "GROUP_RANK": str(self.node_rank)})
            cpus = None
            if self.numa_pin:
                node = gpu_numa_node(local)
                cpus = numa_cpus(node) if node is not None else None

            def _pre(cpus=cpus):
                os.setsid()
                if cpus:
                    try:
                        os.sched_setaffinity(0, cpus)
                    except OSError:
                        pass

            self.procs.append(subprocess.Popen(self.cmd, env=e, preexec_fn=_pre))
        return self

    def wait(self, poll_s: float = 0.2) -> int:
        """Block until all ranks exit; on the first failure tear the others down. Returns the exit code."""
        rc = 0
        live = set(range(self.nproc))
        while live:
            for i in list(live):
                r = self.procs[i].poll()
                if r is None:
                    continue
                live.discard(i)
                if r != 0 and rc == 0:
                    rc = r if r > 0 else 128 - r
                    sys.stderr.write(f"[launch] rank {i} exited with {r}; stopping the other ranks\n")
                    self.terminate(exclude=i)
            time.sleep(poll_s)
        return rc

    def terminate(self, exclude: Optional[int] = None) -> None:
        """SIGTERM each remaining rank's own process group, SIGKILL after the grace period."""
        targets = [p for i, p in enumerate(self.procs) if i != exclude and p.poll() is None]
        for p in targets:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
        t0 = time.time()
        while time.time() - t0 < self.grace_s and any(p.poll() is None for p in targets):
            time.sleep(0.1)
        for p in targets:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="skyrl_b200.launch")
    ap.add_argument("--nproc-per-node", type=int, default=0, help="0 = one per visible GPU")
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--master-addr", default=None)
    ap.add_argument("--master-port", type=int, default=None)
    ap.add_argument("--no-numa-pin", action="store_true")
    ap.add_argument("-m", dest="module", default=None)
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    n = a.nproc_per_node
    if n <= 0:
        try:
            import torch

            n = max(1, torch.cuda.device_count())
        except Exception:
            n = 1
    rest = [x for x in a.rest if x != "--"] if a.rest[:1] == ["--"] else a.rest
    if a.module:
        cmd = [sys.executable, "-m", a.module] + rest
    elif rest:
        cmd = [sys.executable] + rest
    else:
        ap.error("give a module (-m pkg.mod) or a script path")
    env = dict(os.environ)
    if a.master_addr:
        env["MASTER_ADDR"] = a.master_addr
    if a.master_port:
        env["MASTER_PORT"] = str(a.master_port)
    g = WorkerGroup(cmd, n, env=env, numa_pin=not a.no_numa_pin, node_rank=a.node_rank, nnodes=a.nnodes).start()

    def _forward(sig, _frame):
        g.terminate()

    signal.signal(signal.SIGINT, _forward)
    signal.signal(signal.SIGTERM, _forward)
    return g.wait()


if __name__ == "__main__":
    sys.exit(main())
