"""Keep a rank's pinned expert records on the NUMA node its GPU hangs off.

Host-to-device copies of missed experts are the bottleneck of the offloading path; a copy from
memory of the other socket crosses the inter-socket link first and runs at roughly half the PCIe
rate. Pinned pages are placed on the node of the thread that first touches them, so binding the
process to the GPU's node before the records are allocated is enough.
"""
from __future__ import annotations

import os


def _cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(device_index: int) -> int | None:
    """NUMA node of a CUDA device from sysfs, or None when the platform does not say."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, AttributeError, ValueError, RuntimeError, AssertionError):  # also: no CUDA device at all
        return None


def bind_to_gpu_numa_node(device_index: int) -> dict:
    """Restricts this process to the CPUs of the GPU's NUMA node. Returns what was done."""
    node = gpu_numa_node(device_index)
    if node is None:
        return {"numa_node": None, "bound": False}
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = _cpulist(f.read()) & os.sched_getaffinity(0)
        if not cpus:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "bound": True, "cpus": len(cpus)}
    except OSError:
        return {"numa_node": node, "bound": False}
