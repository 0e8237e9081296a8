"""NUMA placement of a rank's host side: the threads of the host Adam, the NVMe workers and
the pinned staging memory (first touch) of a rank belong on the socket its GPU hangs off,
otherwise every gradient and parameter byte of the host share crosses the socket
interconnect twice.  The reference budgets ``cpu_count // world`` threads per rank and
leaves their placement to the OS (flextrain/utils/distributed.py:78-89).

Opt-in (environment variable FLEXTRAIN_NUMA=1, read by ``init_distributed``).  Everything
is read from sysfs; whatever is missing or refused (a VM without NUMA information, a
cpuset that excludes the node) leaves the process as it was.
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Sequence, Set

from .logging import logger


def parse_cpulist(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> [0, 1, 2, 3, 8, 10, 11] (the format of sysfs ``cpulist`` files)."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pci_address(domain: int, bus: int, device: int) -> str:
    return f"{domain:04x}:{bus:02x}:{device:02x}.0"


def gpu_numa_node(pci_addr: str, sysfs: str = "/sys") -> int:
    """NUMA node of the PCI device, -1 when the platform does not say."""
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", pci_addr.lower(), "numa_node")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return -1


def node_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(sysfs, f"devices/system/node/node{node}/cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


def plan_affinity(local_rank: int, gpu_nodes: Sequence[int], allowed: Iterable[int],
                  sysfs: str = "/sys") -> Optional[List[int]]:
    """CPUs for ``local_rank``: those of its GPU's node that the process may use, cut evenly
    among the local ranks whose GPUs share the node.  None when nothing can be said."""
    if not 0 <= local_rank < len(gpu_nodes):
        return None
    node = gpu_nodes[local_rank]
    if node < 0:
        return None
    allowed_set: Set[int] = set(allowed)
    cpus = [c for c in node_cpus(node, sysfs) if c in allowed_set]
    sharers = [r for r, n in enumerate(gpu_nodes) if n == node]
    per = len(cpus) // len(sharers)
    if per == 0:
        return None
    k = sharers.index(local_rank)
    return cpus[k * per:(k + 1) * per]


def local_gpu_nodes(count: int, sysfs: str = "/sys") -> List[int]:
    import torch
    nodes = []
    for i in range(count):
        p = torch.cuda.get_device_properties(i)
        addr = pci_address(getattr(p, "pci_domain_id", 0), getattr(p, "pci_bus_id", 0),
                           getattr(p, "pci_device_id", 0))
        nodes.append(gpu_numa_node(addr, sysfs))
    return nodes


def bind_to_gpu_node(local_rank: int, local_world: int, sysfs: str = "/sys",
                     gpu_nodes: Optional[Sequence[int]] = None) -> Optional[List[int]]:
    """Pin this process (and the threads it starts later) to its share of the CPUs next to
    its GPU and size the thread pools to it.  Returns the CPUs, or None if nothing changed."""
    try:
        import torch
        if gpu_nodes is None:
            if not torch.cuda.is_available():
                return None
            gpu_nodes = local_gpu_nodes(min(local_world, torch.cuda.device_count()), sysfs)
        cpus = plan_affinity(local_rank, gpu_nodes, os.sched_getaffinity(0), sysfs)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        os.environ["OMP_NUM_THREADS"] = str(len(cpus))
        torch.set_num_threads(len(cpus))
        logger.info(f"local rank {local_rank}: bound to {len(cpus)} CPUs of NUMA node {gpu_nodes[local_rank]}")
        return cpus
    except Exception as exc:                       # placement is an optimisation, never a reason to stop
        logger.warning(f"NUMA binding skipped: {type(exc).__name__}: {exc}")
        return None
