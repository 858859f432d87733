"""Host-side placement for the host-buffer path (``PEER.forward_host*``): which CPU cores and which
memory node are local to a GPU, and binding the calling process to them BEFORE its pinned staging
buffers are allocated, so that the DMA engines of the GPU read and write memory on their own socket
and several ranks on one host do not migrate over each other's cores.

Everything here is best effort: on a host that exposes no topology (a container with one visible
memory node, no sysfs) the functions report what they found and change nothing.  Nothing here touches
any GPU setting.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def pci_address(device_index: int) -> Optional[str]:
    """sysfs name (dddd:bb:dd.0) of a CUDA device, or None."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def gpu_locality(device_index: int, sysfs_root: str = "/sys/bus/pci/devices") -> Dict:
    """{"pci": address, "numa_node": int or None, "cpus": cores local to the device or []}."""
    addr = pci_address(device_index)
    info: Dict = {"pci": addr, "numa_node": None, "cpus": []}
    if addr is None:
        return info
    base = os.path.join(sysfs_root, addr)
    node = _read(os.path.join(base, "numa_node"))
    if node is not None:
        try:
            info["numa_node"] = int(node) if int(node) >= 0 else None
        except ValueError:
            pass
    cl = _read(os.path.join(base, "local_cpulist"))
    if cl:
        try:
            info["cpus"] = _parse_cpulist(cl)
        except ValueError:
            pass
    return info


def _set_preferred_node(node: int) -> bool:
    """set_mempolicy(MPOL_PREFERRED, {node}) for this thread and the memory it touches from now on."""
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        MPOL_PREFERRED, SYS_set_mempolicy = 1, 238          # x86-64
        if os.uname().machine != "x86_64":
            return False
        mask = ctypes.c_ulong(1 << node)
        rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(node + 2))
        return rc == 0
    except Exception:
        return False


def slice_for_rank(cpus: List[int], local_rank: int, local_world: int) -> List[int]:
    """The share of a core list that rank `local_rank` of `local_world` ranks on this host keeps: ranks
    whose GPUs report the same local cores split them evenly instead of all floating over all."""
    if local_world <= 1 or len(cpus) < local_world:
        return list(cpus)
    per = len(cpus) // local_world
    return cpus[local_rank * per:(local_rank + 1) * per]


def bind_process_to_gpu(device_index: int, local_rank: int = 0, local_world: int = 1,
                        sysfs_root: str = "/sys/bus/pci/devices") -> Dict:
    """Pin this process to (its share of) the cores local to the GPU and prefer the GPU's memory node
    for later allocations.  Call before allocating pinned buffers.  Returns what was found and done."""
    info = gpu_locality(device_index, sysfs_root)
    done = {"pci": info["pci"], "numa_node": info["numa_node"], "cpus_bound": None, "mempolicy": False}
    try:
        allowed = sorted(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return done
    local = [c for c in info["cpus"] if c in allowed] or allowed
    share = slice_for_rank(local, local_rank, local_world)
    if share:
        try:
            os.sched_setaffinity(0, share)
            done["cpus_bound"] = f"{share[0]}-{share[-1]} ({len(share)} cores)"
        except OSError:
            pass
    if info["numa_node"] is not None:
        done["mempolicy"] = _set_preferred_node(info["numa_node"])
    return done


def pinned_empty(*shape, dtype=torch.float32) -> torch.Tensor:
    """A pinned host tensor, allocated (and therefore placed) by the calling thread under whatever
    affinity and memory policy `bind_process_to_gpu` set."""
    return torch.empty(*shape, dtype=dtype, pin_memory=True)
