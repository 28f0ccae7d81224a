"""Host-memory placement for the pinned buffers that feed a GPU.

Eight ranks that each copy tens of megabytes per step from pinned host memory are limited by
where those pages live: a buffer on the far socket crosses the inter-socket link on every
copy. The reference's harness binds each rank to the NUMA node of its GPU before it allocates
and verifies the placement from ``/proc/self/numa_maps`` (benchmarks/communication.py:66-78 of
the reference). This module does the same with plain files and system calls:

* ``device_numa_node`` reads the node of a GPU from its PCI device directory;
* ``bind_to_device`` restricts the calling process to that node's CPUs (new pinned pages then
  land there by first touch) and asks the kernel to prefer the node for its memory;
* ``pages_by_node`` reports where the pages of an address range actually are.

Containers often hide the PCI tree of sysfs; the driver still knows the topology, so when
sysfs gives no node the ideal CPU set of the GPU is read from NVML (a read-only query) and the
process is bound to those CPUs instead.

Everything degrades to a no-op (and says so in the returned record) on machines without NUMA
information, inside containers that hide it, or where the calls are not permitted.
"""

from __future__ import annotations

import ctypes
import os
import platform
from typing import Dict, List, Optional

_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}
_MPOL_PREFERRED = 1


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]``."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            first, last = part.split("-", 1)
            cpus.extend(range(int(first), int(last) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pci_address(domain: int, bus: int, device: int) -> str:
    return f"{domain:04x}:{bus:02x}:{device:02x}.0"


def device_pci_address(device_index: int) -> Optional[str]:
    import torch
    props = torch.cuda.get_device_properties(device_index)
    try:
        return pci_address(props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except AttributeError:
        return None


def node_of_pci_device(address: Optional[str], sysfs: str = "/sys") -> int:
    """NUMA node of a PCI device, or -1 when the platform does not say."""
    if not address:
        return -1
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", address, "numa_node")) as handle:
            return int(handle.read().strip())
    except (OSError, ValueError):
        return -1


def device_numa_node(device_index: int, sysfs: str = "/sys") -> int:
    return node_of_pci_device(device_pci_address(device_index), sysfs)


def node_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(sysfs, f"devices/system/node/node{node}/cpulist")) as handle:
            return parse_cpu_list(handle.read())
    except OSError:
        return []


def prefer_node(node: int) -> bool:
    """Ask the kernel to allocate this thread's future pages on ``node`` first. Best effort."""
    number = _SET_MEMPOLICY.get(platform.machine())
    if number is None or not 0 <= node < 1024:
        return False
    words = node // 64 + 1
    mask = (ctypes.c_ulong * words)()
    mask[node // 64] = 1 << (node % 64)
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        return libc.syscall(number, _MPOL_PREFERRED, mask, ctypes.c_ulong(words * 64 + 1)) == 0
    except (OSError, AttributeError):
        return False


def bind_to_node(node: int, sysfs: str = "/sys", *, set_affinity=os.sched_setaffinity,
                 get_affinity=os.sched_getaffinity, prefer=prefer_node) -> Dict[str, object]:
    """Run on the CPUs of ``node`` (within the current affinity mask) and prefer its memory."""
    record: Dict[str, object] = {"node": node, "bound": False, "cpus": 0, "memory_policy": False}
    if node < 0:
        record["reason"] = "the platform reports no NUMA node for the device"
        return record
    allowed = set(get_affinity(0))
    cpus = sorted(allowed.intersection(node_cpus(node, sysfs)))
    if not cpus:
        record["reason"] = "none of the node's CPUs is in this process's affinity mask"
        return record
    try:
        set_affinity(0, cpus)
    except OSError as error:
        record["reason"] = f"sched_setaffinity failed: {error}"
        return record
    record.update(bound=True, cpus=len(cpus), memory_policy=bool(prefer(node)))
    return record


def nvml_cpu_affinity(address: Optional[str], nvml=None) -> List[int]:
    """CPUs the driver considers closest to the GPU at PCI ``address`` (empty when unknown)."""
    if not address:
        return []
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
        handle = nvml.nvmlDeviceGetHandleByPciBusId(address.encode() if isinstance(address, str) else address)
        words = (os.cpu_count() or 64) // 64 + 1
        mask = nvml.nvmlDeviceGetCpuAffinity(handle, words)
    except Exception:
        return []
    return [word * 64 + bit for word, value in enumerate(mask) for bit in range(64) if (int(value) >> bit) & 1]


def bind_to_cpus(cpus, *, set_affinity=os.sched_setaffinity, get_affinity=os.sched_getaffinity) -> Dict[str, object]:
    """Run on ``cpus`` (within the current affinity mask); memory then follows by first touch."""
    record: Dict[str, object] = {"node": -1, "bound": False, "cpus": 0, "memory_policy": False, "source": "nvml"}
    chosen = sorted(set(get_affinity(0)).intersection(cpus))
    if not chosen:
        record["reason"] = "no CPU near the device is known, or none is in this process's affinity mask"
        return record
    try:
        set_affinity(0, chosen)
    except OSError as error:
        record["reason"] = f"sched_setaffinity failed: {error}"
        return record
    record.update(bound=True, cpus=len(chosen))
    return record


def bind_to_device(device_index: int, sysfs: str = "/sys", *, nvml=None) -> Dict[str, object]:
    """Bind the calling process to the NUMA node of CUDA device ``device_index``.

    Call it before allocating pinned host memory. Returns a record for the benchmark report:
    ``{"node", "bound", "cpus", "memory_policy"[, "reason"][, "source"]}``.
    """
    address = device_pci_address(device_index)
    node = node_of_pci_device(address, sysfs)
    if node >= 0:
        return bind_to_node(node, sysfs)
    return bind_to_cpus(nvml_cpu_affinity(address, nvml))


def pages_by_node(address: int, maps_path: str = "/proc/self/numa_maps") -> Dict[int, int]:
    """Pages per NUMA node of the mapping that starts at or contains ``address``.

    ``numa_maps`` lists one mapping per line: its start address in hex, the policy, then
    ``N<node>=<pages>`` items. A pinned allocation is one mapping (or the tail of one), so the
    mapping with the greatest start that is not above the address is the one reported.
    """
    best_start = -1
    best: Dict[int, int] = {}
    try:
        with open(maps_path) as handle:
            for line in handle:
                fields = line.split()
                if not fields:
                    continue
                try:
                    start = int(fields[0], 16)
                except ValueError:
                    continue
                if start <= address and start > best_start:
                    best_start = start
                    best = {int(item[1:].split("=")[0]): int(item.split("=")[1])
                            for item in fields[1:] if item.startswith("N") and "=" in item and item[1].isdigit()}
    except OSError:
        return {}
    return best
