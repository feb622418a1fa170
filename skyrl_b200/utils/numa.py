"""Pin a rank's host threads to the CPUs next to its GPU.

The reference binds each worker to the NUMA node of its GPU through libnuma (``DistributedTorchRayActor``,
skyrl/backends/skyrl_train/workers/worker.py, NUMA pinning via ctypes).  Here the topology is read from sysfs
(``/sys/bus/pci/devices/<bus id>/numa_node`` and ``/sys/devices/system/node/node<N>/cpulist``) and applied with
``os.sched_setaffinity``: no native dependency, and a no-op wherever the files are absent (containers, single-node
hosts).  Pinned host memory for the H2D input copies and the engine's scheduler thread then sit on the GPU's node.
"""

from __future__ import annotations

import os
from typing import List, Optional


def parse_cpulist(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]``."""
    out: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


def gpu_numa_node(pci_bus_id: str, sysfs_root: str = "/sys") -> Optional[int]:
    """NUMA node of a PCI device (``0000:1b:00.0``); ``None`` when unknown (file missing or ``-1``)."""
    path = os.path.join(sysfs_root, "bus", "pci", "devices", pci_bus_id.lower(), "numa_node")
    try:
        with open(path) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs_root: str = "/sys") -> List[int]:
    path = os.path.join(sysfs_root, "devices", "system", "node", f"node{node}", "cpulist")
    try:
        with open(path) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def _bus_id_of(device_index: int) -> Optional[str]:
    try:
        import torch

        if not torch.cuda.is_available():
            return None
        props = torch.cuda.get_device_properties(device_index)
        dom = getattr(props, "pci_domain_id", 0)
        return f"{dom:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    except Exception:
        return None


def pin_to_gpu_numa_node(device_index: int, sysfs_root: str = "/sys", bus_id: Optional[str] = None,
                         setaffinity=os.sched_setaffinity) -> List[int]:
    """Restrict the calling process to the CPUs of the GPU's NUMA node; returns the CPU list applied (empty = unchanged)."""
    bus_id = bus_id or _bus_id_of(device_index)
    if not bus_id:
        return []
    node = gpu_numa_node(bus_id, sysfs_root)
    if node is None:
        return []
    cpus = node_cpus(node, sysfs_root)
    if hasattr(os, "sched_getaffinity"):
        allowed = os.sched_getaffinity(0)
        cpus = [c for c in cpus if c in allowed] if setaffinity is os.sched_setaffinity else cpus
    if not cpus:
        return []
    setaffinity(0, set(cpus))
    return cpus
