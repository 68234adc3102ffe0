"""Host-side placement of a rank next to its GPU.

With one process per GPU on a two-socket host, pinned host buffers land on the NUMA node of the thread that first
touches them.  A rank whose buffers sit on the other socket pays an inter-socket hop for every byte its GPU reads or
writes over PCIe; with eight ranks streaming results to the host at once that hop is the bottleneck.  Binding the
process to the CPUs of the GPU's own NUMA node (before anything is allocated) keeps those copies local.  Only this
process's CPU affinity is changed; nothing about the GPU or the machine is.
"""
import os
from typing import Optional

import torch


def _cpulist(text: str):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(device_index: int) -> Optional[int]:
    """NUMA node of the GPU's PCIe slot, or None when the platform does not tell."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def bind_to_gpu_numa_node(device_index: int) -> dict:
    """Restrict this process to the CPUs of the GPU's NUMA node (intersected with the CPUs it is allowed to use).
    Returns what was done: ``{"numa_node": n or None, "cpus": number of CPUs the process may use afterwards}``."""
    node = gpu_numa_node(device_index)
    info = {"numa_node": node, "cpus": len(os.sched_getaffinity(0))}
    if node is None:
        return info
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            local = _cpulist(f.read())
        allowed = os.sched_getaffinity(0) & local
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["cpus"] = len(allowed)
    except Exception:
        pass
    return info
