"""Keep a rank's host memory next to its GPU.

A pinned buffer is placed on the NUMA node of the thread that allocates it. With one process per GPU and no binding, every
rank's staging buffers can end up on one socket: host-to-device copies of the GPUs behind the other socket then cross the
inter-socket link and all of them share one socket's memory channels. ``bind_to_gpu(i)`` moves the calling process to the
CPUs of GPU i's node and makes that node the preferred one for new pages; call it before allocating pinned memory.
Everything is read from sysfs; where the information is missing (containers without /sys, single-node hosts) it is a no-op."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Set


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def parse_cpulist(text: str) -> Set[int]:
    """"0-3,8,10-11" -> {0, 1, 2, 3, 8, 10, 11}."""
    cpus: Set[int] = set()
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_pci_address(index: int) -> Optional[str]:
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:  # noqa: BLE001  (no CUDA, or a torch without the PCI fields)
        return None


def gpu_numa_node(index: int, sysfs: str = "/sys") -> Optional[int]:
    addr = gpu_pci_address(index)
    if addr is None:
        return None
    text = _read(f"{sysfs}/bus/pci/devices/{addr}/numa_node")
    if text is None:
        return None
    try:
        node = int(text)
    except ValueError:
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> Set[int]:
    text = _read(f"{sysfs}/devices/system/node/node{node}/cpulist")
    return parse_cpulist(text) if text else set()


def prefer_node(node: int) -> bool:
    """set_mempolicy(MPOL_PREFERRED, {node}) for the calling thread: new pages come from ``node`` while it has room."""
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        words = node // 64 + 1
        mask = (ctypes.c_ulong * words)()
        mask[node // 64] = 1 << (node % 64)
        sys_set_mempolicy = {"x86_64": 238, "aarch64": 237}.get(os.uname().machine)
        if sys_set_mempolicy is None:
            return False
        return libc.syscall(sys_set_mempolicy, 1, ctypes.byref(mask), ctypes.c_ulong(words * 64 + 1)) == 0
    except Exception:  # noqa: BLE001
        return False


def bind_to_gpu(index: int, sysfs: str = "/sys") -> dict:
    """Moves this process next to GPU ``index``. -> {"node": n or None, "cpus": how many CPUs it now runs on, "mempolicy": bool}."""
    node = gpu_numa_node(index, sysfs)
    out = {"node": node, "cpus": len(os.sched_getaffinity(0)), "mempolicy": False}
    if node is None:
        return out
    cpus = node_cpus(node, sysfs) & os.sched_getaffinity(0)
    if cpus:
        try:
            os.sched_setaffinity(0, cpus)
            out["cpus"] = len(cpus)
        except OSError:
            pass
    out["mempolicy"] = prefer_node(node)
    return out
