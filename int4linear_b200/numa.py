"""Host-side placement for the host-buffer entry point (int4_linear_host).

The reference's correctness program stages its operands through pageable host memory of whatever
NUMA node the process happens to run on (test/test_correctness.cu:38-58).  With one process per
GPU on a multi-socket host, pinned staging buffers that sit on the far socket halve the PCIe copy
rate and make the ranks compete for one socket's memory bandwidth.  Linux places a page on the
node of the CPU that first touches it, so running the process on the CPUs of the GPU's own node
BEFORE it allocates and pins its buffers is enough.

    bind_to_gpu_node(pci_bus_id)   restrict this process to the CPUs next to that GPU

Everything here only reads /sys and calls sched_setaffinity on the calling process; nothing about
the GPU or the machine is changed.
"""
from __future__ import annotations

import os


def parse_cpulist(text: str) -> set[int]:
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11}"""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> int | None:
    """NUMA node of the PCI device 'dddd:bb:dd.f' (None when the kernel reports none)."""
    path = os.path.join(sysfs, "bus", "pci", "devices", pci_bus_id.lower(), "numa_node")
    try:
        with open(path) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> set[int]:
    try:
        with open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return set()


def bind_to_gpu_node(pci_bus_id: str, sysfs: str = "/sys", setaffinity=None, allowed: set[int] | None = None) -> dict:
    """Restrict the calling process to the CPUs of the NUMA node the GPU hangs off, keeping only
    CPUs it is allowed to use already.  Returns what was done: {"node": n or None, "cpus": count,
    "bound": bool}.  `setaffinity` / `allowed` exist for tests."""
    node = gpu_numa_node(pci_bus_id, sysfs)
    if node is None:
        return {"node": None, "cpus": 0, "bound": False}
    if allowed is None:
        allowed = set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else set()
    cpus = node_cpus(node, sysfs) & allowed
    if not cpus:
        return {"node": node, "cpus": 0, "bound": False}
    try:
        (setaffinity or (lambda c: os.sched_setaffinity(0, c)))(cpus)
    except OSError:
        return {"node": node, "cpus": len(cpus), "bound": False}
    return {"node": node, "cpus": len(cpus), "bound": True}


def torch_pci_bus_id(device_index: int) -> str | None:
    """PCI address of a CUDA device as sysfs spells it, from torch's device properties."""
    import torch
    p = torch.cuda.get_device_properties(device_index)
    try:
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except AttributeError:
        return None
