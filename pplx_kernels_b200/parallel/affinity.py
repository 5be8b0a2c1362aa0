"""CPU and host-memory placement of a rank next to its GPU.

A rank's pinned staging buffers are read and written by its GPU over PCIe.  On a
two-socket host the copy crosses the socket interconnect whenever the pages sit on
the other socket, and with eight ranks copying at once that link, not PCIe, sets
the pace.  ``bind_to_device_numa_node`` restricts the calling process to the CPUs
of the NUMA node the GPU hangs off, *before* pinned memory is allocated, so that
the default first-touch policy places the pages locally.  Only the process's own
CPU affinity changes; nothing of the GPU or the host is configured.

The reference leaves placement to the launcher (its benchmark is started by
``mp.spawn`` with no binding: tests/distributed_utils.py:55-118).
"""

from __future__ import annotations

import os
from pathlib import Path


def parse_cpulist(text: str) -> set[int]:
    """``"0-3,8,10-11"`` -> {0, 1, 2, 3, 8, 10, 11} (the sysfs cpulist format)."""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def pci_address(domain: int, bus: int, device: int) -> str:
    """sysfs name of PCI function 0 of a device."""
    return f"{domain:04x}:{bus:02x}:{device:02x}.0"


def device_local_cpus(pci_addr: str, sysfs_root: str | os.PathLike = "/sys") -> set[int]:
    """CPUs that are local to the PCI device, or an empty set when sysfs does not say."""
    base = Path(sysfs_root) / "bus" / "pci" / "devices" / pci_addr
    try:
        cpus = parse_cpulist((base / "local_cpulist").read_text())
    except (OSError, ValueError):
        cpus = set()
    if cpus:
        return cpus
    try:
        node = int((base / "numa_node").read_text().strip())
        if node < 0:
            return set()
        text = (Path(sysfs_root) / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text()
        return parse_cpulist(text)
    except (OSError, ValueError):
        return set()


def bind_to_device_numa_node(device_index: int, sysfs_root: str | os.PathLike = "/sys") -> dict:
    """Restricts this process to the CPUs local to CUDA device ``device_index``.

    Returns what was done: ``{"bound": bool, "cpus": n, "pci": "...", "reason": "..."}``.
    Never raises: with no topology information, a single node, or an affinity mask that
    the container does not allow, the process is left as it was.
    """
    info: dict = {"bound": False, "cpus": 0, "pci": None, "reason": ""}
    try:
        import torch

        props = torch.cuda.get_device_properties(device_index)
        addr = pci_address(int(props.pci_domain_id), int(props.pci_bus_id), int(props.pci_device_id))
    except Exception as exc:  # noqa: BLE001 - placement is best effort
        info["reason"] = f"no PCI address: {type(exc).__name__}"
        return info
    info["pci"] = addr
    local = device_local_cpus(addr, sysfs_root)
    if not local:
        info["reason"] = "sysfs gives no local CPUs for the device"
        return info
    try:
        allowed = os.sched_getaffinity(0)
        target = local & allowed
        if not target:
            info["reason"] = "local CPUs are outside the allowed set"
            return info
        if target == allowed:
            info["reason"] = "already local"
            info["cpus"] = len(target)
            return info
        os.sched_setaffinity(0, target)
    except (OSError, AttributeError) as exc:
        info["reason"] = f"affinity call failed: {type(exc).__name__}"
        return info
    info["bound"] = True
    info["cpus"] = len(target)
    return info
