"""Host-side placement for a one-process-per-GPU job: keep a rank's threads, and with them the pages of the pinned
staging buffers it allocates afterwards (first touch), on the NUMA node its GPU hangs off.

Every rank of the data-parallel MLP step copies its rows of the batch from pinned host memory every step. On a
two-socket host, eight ranks whose buffers all sit on the node the launcher happened to run on pull everything
through one socket's memory controllers and the inter-socket link; bound to their GPU's node, each socket serves
only its own four GPUs. Nothing here touches the device or any setting that outlasts the process.

The reference has no multi-device or host-memory code (device hard-wired to 0, src/python_bindings/bindings.cpp:123;
torch owns every buffer), so nothing here mirrors a reference interface.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import List, Optional

SYSFS = Path("/sys")


def parse_cpulist(text: str) -> List[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11] (the kernel's cpulist format); '' -> []."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            lo_i, hi_i = int(lo), int(hi)
            if hi_i < lo_i:
                raise ValueError(f"bad cpulist range {part!r}")
            cpus.extend(range(lo_i, hi_i + 1))
        else:
            cpus.append(int(part))
    return sorted(set(cpus))


def numa_node_of_pci(bus_id: str, sysfs: Path = SYSFS) -> Optional[int]:
    """NUMA node of a PCI device ('0000:1b:00.0', any case), or None when the host does not say (single node, -1)."""
    f = sysfs / "bus" / "pci" / "devices" / bus_id.strip().lower() / "numa_node"
    try:
        node = int(f.read_text().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def cpus_of_node(node: int, sysfs: Path = SYSFS) -> List[int]:
    try:
        return parse_cpulist((sysfs / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text())
    except (OSError, ValueError):
        return []


def device_pci_bus_id(device: int) -> str:
    import ctypes as C
    from ._lib import check, lib
    buf = C.create_string_buffer(32)
    check(lib.aicf_b200_device_pci_bus_id(device, buf, len(buf)), "device_pci_bus_id")
    return buf.value.decode()


def bind_to_device_node(device: int, *, bus_id: Optional[str] = None, sysfs: Path = SYSFS,
                        setaffinity=None, allowed=None) -> dict:
    """Restricts the calling thread, and with it the threads it starts afterwards, to the CPUs of the NUMA node of
    `device` (intersected with the CPUs it may already use; threads that already exist keep their own masks). Call it
    from the thread that allocates the pinned buffers, before it does so. Returns what it found and did; does nothing, and says why, when the
    host does not expose a node, the node has no CPU the process may use, or AICF_HOST_AFFINITY=0."""
    info = {"device": device, "bus_id": None, "numa_node": None, "cpus": None, "bound": False, "why_not": None}
    if os.environ.get("AICF_HOST_AFFINITY", "1") == "0":
        info["why_not"] = "AICF_HOST_AFFINITY=0"
        return info
    setaffinity = setaffinity or getattr(os, "sched_setaffinity", None)
    if allowed is None:
        getaff = getattr(os, "sched_getaffinity", None)
        allowed = set(getaff(0)) if getaff else None
    if setaffinity is None or allowed is None:
        info["why_not"] = "no sched_setaffinity on this platform"
        return info
    info["bus_id"] = bus_id if bus_id is not None else device_pci_bus_id(device)
    node = numa_node_of_pci(info["bus_id"], sysfs)
    if node is None:
        info["why_not"] = "host reports no NUMA node for the device"
        return info
    info["numa_node"] = node
    cpus = sorted(set(cpus_of_node(node, sysfs)) & set(allowed))
    if not cpus:
        info["why_not"] = "the node has no CPU this process may run on"
        return info
    setaffinity(0, cpus)
    info["cpus"] = len(cpus)
    info["bound"] = True
    return info
