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


def _gpu_bdf(device_index: int) -> str | None:
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except (AttributeError, ValueError, RuntimeError, AssertionError):  # also: no CUDA device at all
        return None


def gpu_numa_node(device_index: int, sysfs: str = "/sys") -> int | None:
    """NUMA node of a CUDA device from sysfs, or None when the platform does not say."""
    bdf = _gpu_bdf(device_index)
    if bdf is None:
        return None
    try:
        with open(f"{sysfs}/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError):
        return None


def gpu_local_cpus(device_index: int, sysfs: str = "/sys") -> set[int]:
    """CPUs the PCI device reports as local (`local_cpulist`), empty when unknown. Virtualised hosts
    often report numa_node -1 and still fill this list."""
    bdf = _gpu_bdf(device_index)
    if bdf is None:
        return set()
    try:
        with open(f"{sysfs}/bus/pci/devices/{bdf}/local_cpulist") as f:
            return _cpulist(f.read())
    except (OSError, ValueError):
        return set()


def bind_to_gpu_numa_node(device_index: int, sysfs: str = "/sys") -> dict:
    """Restricts this process to the CPUs next to the GPU: those of its NUMA node, or, when the
    platform reports no node (numa_node = -1), the device's local_cpulist if that is a proper
    subset of the CPUs the process may use. Returns what was done."""
    allowed = os.sched_getaffinity(0)
    node = gpu_numa_node(device_index, sysfs)
    try:
        if node is not None:
            with open(f"{sysfs}/devices/system/node/node{node}/cpulist") as f:
                cpus, source = _cpulist(f.read()) & allowed, "numa_node"
        else:
            cpus, source = gpu_local_cpus(device_index, sysfs) & allowed, "local_cpulist"
            if cpus == allowed:  # the device is local to everything this process can use: one node, nothing to do
                return {"numa_node": None, "bound": False, "reason": "no locality information (single node)"}
        if not cpus:
            return {"numa_node": node, "bound": False, "reason": "no usable CPU listed"}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "bound": True, "cpus": len(cpus), "source": source}
    except OSError:
        return {"numa_node": node, "bound": False, "reason": "sysfs not readable"}
